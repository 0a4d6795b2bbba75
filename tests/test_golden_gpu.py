"""The engine against EmersonDowell/AIR's own logits, without the plain implementation in between: the
golden files under tests/golden/ hold, for the two tiny configurations of the tests, random weights, a token
sequence and the logits that AIR's compiled CPU executor (src/reference/reference_executor.cpp:325-428) gave
for it token by token.  The engine reads the same weights from a model folder and must reproduce the logits
whole, token by token and in portions, in float32, to a few units of rounding.  (The golden models are drawn
with large weights, attention scores of a standard deviation above 10: softmax is all but one-hot there, and
bfloat16 rounding moves logits by more than any tolerance that would still mean something.  The bfloat16 path
is compared with the plain implementation on the replay suite's models, and the plain implementation with
AIR's logits in tests/test_plain.py.)"""
import os
import tempfile

import numpy as np
import pytest
import torch

import util
from golden.make_golden import CONFIGS, from_bf16_bits

pytestmark = pytest.mark.gpu

_folders = {}


def golden_folder(which):
    """config.json and model.safetensors (bfloat16, which holds the golden weights exactly) for a golden file."""
    if which not in _folders:
        from air_b200.weights.loader import write_model_folder
        config, _, file_name = CONFIGS[which]
        z = np.load(os.path.join(util.ROOT, "tests", "golden", file_name))
        tensors = {}
        for i, name in enumerate(str(n) for n in z["names"]):
            values = torch.from_numpy(from_bf16_bits(z[f"w{i}"]).reshape(tuple(z[f"s{i}"])).copy())
            tensors[name] = values.to(torch.bfloat16)
            assert torch.equal(tensors[name].float(), values)
        d = tempfile.TemporaryDirectory(prefix=f"air_b200_golden_{which}_")
        write_model_folder(d.name, config, tensors)
        _folders[which] = (d, z["tokens"].tolist(), z["logits"])
    d, tokens, logits = _folders[which]
    return d.name, tokens, logits


@pytest.mark.parametrize("which", ["a", "b"])
def test_engine_reproduces_air_logits(which, dtype="float32"):
    from air_b200.engine.batch import Entry
    from air_b200.engine.engine import Engine, EngineConfig
    folder, tokens, want = golden_folder(which)
    engine = Engine.from_folder(folder, EngineConfig(dtype=dtype, page_tokens=16, max_tokens=256))
    n = len(tokens)
    whole = engine.step([Entry("whole", tokens, range(n))]).cpu().numpy()
    single = np.concatenate([engine.step([Entry("single", [t], [0])]).cpu().numpy() for t in tokens])
    cut = np.concatenate([engine.step([Entry("cut", tokens[:17], range(17))]).cpu().numpy(),
                          engine.step([Entry("cut", tokens[17:19], range(2))]).cpu().numpy(),
                          engine.step([Entry("cut", tokens[19:], range(n - 19))]).cpu().numpy()])
    engine.check_status()
    scale = max(1.0, float(np.abs(want).max()))
    for got in (whole, single, cut):
        diff = np.abs(got - want)
        assert diff.max() <= util.FP32_TOL * scale, float(diff.max())
        assert (got.argmax(-1) == want.argmax(-1)).all()
    assert np.array_equal(whole, single) and np.array_equal(whole, cut)
