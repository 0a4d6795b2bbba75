"""Python faces of the CUDA kernels.  Every function checks what it is given (device,
dtype, shape, contiguity), launches on torch's current stream and raises on any error
code.  There is no other implementation behind these functions: if the library cannot be
built or loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_SIGNATURES = {
    "air_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "air_add_parts": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p],
    "air_add_prenorm": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_logits_post": [c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p],
    "air_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                        c_longlong, c_float, c_void_p],
    "air_qkv_rope_store": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "air_silu_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "air_convert": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
    "air_gemm_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "air_paged_attention_ref": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "air_table_update": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_decode_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "air_prefill_attention": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "air_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "air_gemm_tc_small": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p, c_int, c_float, c_void_p],
    "air_decode_attention_tma": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                 c_void_p],
    "air_decode_attention_tma_fresh": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "air_prefill_attention_tc": [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                 c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "air_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                   c_void_p, c_void_p],
}

_fn = {}
launches = 0   # kernels of this library launched so far (each wrapper launches one)


class KernelError(RuntimeError):
    pass


def _get(name):
    f = _fn.get(name)
    if f is None:
        lib = build.library()
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn[name] = f
    return f


def set_pdl(on: bool) -> None:
    """Whether kernels are launched so that they may overlap the tail of their predecessor."""
    lib = build.library()
    lib.air_set_pdl.argtypes = [c_int]
    lib.air_set_pdl.restype = None
    lib.air_set_pdl(1 if on else 0)


TRACE_NAMES = {1: "embedding", 2: "add_rmsnorm", 3: "qkv_rope_store", 4: "silu_mul", 5: "convert", 6: "table_update",
               7: "attention_ref", 8: "decode_attention", 9: "decode_combine", 10: "prefill_attention", 11: "gemm_f32",
               12: "gemm_tc", 13: "sample"}


def set_trace(buffer: Optional[torch.Tensor]) -> None:
    """buffer: int64 CUDA tensor of 1 + 2 * 16384 elements (zeroed), or None to stop tracing.  While set,
    block 0 of every kernel appends (kernel id, GPU nanosecond timer) after its wait on its predecessor;
    element 0 counts the entries.  Differences of consecutive times are the kernels' spans in a graph."""
    lib = build.library()
    ptr = None if buffer is None else buffer.data_ptr()
    for src in build.sources():
        f = getattr(lib, "air_trace_set_" + src[:-3])
        f.argtypes, f.restype = [c_void_p], c_int
        rc = f(ptr)
        if rc:
            raise KernelError(f"set_trace: CUDA error {rc}")


def _check(code: int, name: str):
    global launches
    launches += 1
    if code != 0:
        if code == 100001:
            raise KernelError(f"{name}: a size or dtype that the kernel does not take")
        raise KernelError(f"{name}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream() -> int:
    """The current stream's handle (the stream that a graph capture or a stream context has made current).
    A step launches hundreds of kernels from Python, so this asks the runtime directly where it can."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _req(t: torch.Tensor, name: str, dtypes=None, shape=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise KernelError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if shape is not None:
        got = t.shape
        if len(got) != len(shape):
            raise KernelError(f"{name} has shape {tuple(got)}, expected {tuple(shape)}")
        for s, g in zip(shape, got):
            if s is not None and s != g:
                raise KernelError(f"{name} has shape {tuple(got)}, expected {tuple(shape)}")
    return t


_FLOATS = (torch.float32, torch.bfloat16)
_I32 = (torch.int32,)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def embedding(table, ids, out, status=None, last_token=None, multiplier=1.0):
    """out[t] = table[ids[t]] * multiplier as float32; an id -(s+1) is replaced by last_token[s]."""
    V, E = table.shape
    _req(table, "table", _FLOATS)
    _req(ids, "ids", _I32, (out.shape[0],))
    _req(out, "out", (torch.float32,), (None, E))
    if last_token is not None:
        _req(last_token, "last_token", _I32)
    _check(_get("air_embedding")(table.data_ptr(), _DT[table.dtype], ids.data_ptr(), _ptr(last_token),
                                 out.data_ptr(), out.shape[0], E, V, float(multiplier), _ptr(status), _stream()),
           "embedding")
    return out


def add_parts(h, delta):
    """h += delta in place (float32 h [T, E]); delta [T, E] or partial sums [parts, T, E], added in order."""
    _req(h, "h", (torch.float32,))
    parts = 1 if delta.dim() == h.dim() else delta.shape[0]
    _req(delta, "delta", _FLOATS, tuple(h.shape) if delta.dim() == h.dim() else (parts,) + tuple(h.shape))
    _check(_get("air_add_parts")(h.data_ptr(), delta.data_ptr(), _DT[delta.dtype], parts, h.numel(), _stream()),
           "add_parts")
    return h


PRENORM_CHUNK = 512


def add_prenorm(h, delta, weight, xg, ss):
    """h += delta in place (float32 h [T, E]; delta None, [T, E] or partial sums [parts, T, E]); xg =
    bfloat16(h * weight); ss[chunk, t] = the sum of h[t]^2 over a chunk of 512 columns.  What add_rmsnorm does, short
    of the scale per row (rsqrt(sum of a row's ss / E + eps)), which the product that takes xg applies (gemm_tc's
    row_ss): no block of this kernel waits for another."""
    T, E = h.shape
    _req(h, "h", (torch.float32,))
    parts = 0
    if delta is not None:
        parts = 1 if delta.dim() == 2 else delta.shape[0]
        _req(delta, "delta", _FLOATS, (T, E) if delta.dim() == 2 else (parts, T, E))
    _req(weight, "weight", _FLOATS, (E,))
    _req(xg, "xg", (torch.bfloat16,), (T, E))
    _req(ss, "ss", (torch.float32,), (-(-E // PRENORM_CHUNK), T))
    if E % 4:
        raise KernelError(f"add_prenorm: width {E} is not a multiple of 4")
    _check(_get("air_add_prenorm")(h.data_ptr(), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, parts,
                                   weight.data_ptr(), _DT[weight.dtype], xg.data_ptr(), ss.data_ptr(), T, E,
                                   _stream()), "add_prenorm")
    return xg, ss


def logits_post(logits, bias=None, scale=1.0, softcap=0.0):
    """In place: logits = (logits + bias) * scale, then softcap * tanh(logits / softcap) where softcap > 0."""
    R, V = logits.shape
    _req(logits, "logits", (torch.float32,))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (V,))
    _check(_get("air_logits_post")(logits.data_ptr(), _ptr(bias), float(scale), float(softcap), R, V, _stream()),
           "logits_post")
    return logits


def add_rmsnorm(h, delta, weight, eps, out, rows=None):
    """Without rows: h += delta (in place, float32), out = rmsnorm(h) * weight.
    With rows: out[r] = rmsnorm(h[rows[r]] + delta[rows[r]]) * weight, h unchanged."""
    E = h.shape[-1]
    _req(h, "h", (torch.float32,), (None, E))
    parts = 0
    if delta is not None:
        # [rows, E], or [parts, rows, E]: partial sums that are added in order
        parts = 1 if delta.dim() == 2 else delta.shape[0]
        _req(delta, "delta", _FLOATS, tuple(h.shape) if delta.dim() == 2 else (parts,) + tuple(h.shape))
    _req(weight, "weight", _FLOATS, (E,))
    R = h.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", _I32)
    _req(out, "out", _FLOATS, (R, E))
    _check(_get("air_add_rmsnorm")(h.data_ptr(), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, parts,
                                   weight.data_ptr(), _DT[weight.dtype], out.data_ptr(), _DT[out.dtype],
                                   _ptr(rows), R, E, h.shape[0], float(eps), _stream()), "add_rmsnorm")
    return out


def qkv_rope_store(qkv, bias, table, positions, token_seq, block_table, q_out, cache, heads, kv_heads,
                   head_dim, write_kv=True, status=None):
    """Adds the bias, rotates q and k by the table's cos/sin of each token's position, writes
    q to q_out [T, H, d] and k, v into the pages (cache [page, 2, K, P, d])."""
    T = qkv.shape[-2]
    width = (heads + 2 * kv_heads) * head_dim
    parts = 1 if qkv.dim() == 2 else qkv.shape[0]     # [T, width], or [parts, T, width] partial sums
    _req(qkv, "qkv", _FLOATS, (T, width) if qkv.dim() == 2 else (parts, T, width))
    if bias is not None:
        _req(bias, "bias", _FLOATS, (width,))
    rot = 0
    if table is not None:
        _req(table, "table", (torch.float32,))
        rot = table.shape[1]
        if rot > head_dim or rot % 2:
            raise KernelError(f"rotary width {rot} does not fit head size {head_dim}")
    _req(positions, "positions", _I32, (T,))
    _req(token_seq, "token_seq", _I32, (T,))
    _req(block_table, "block_table", _I32)
    _req(q_out, "q_out", _FLOATS, (T, heads, head_dim))
    _req(cache, "cache", (q_out.dtype,), (None, 2, kv_heads, None, head_dim))
    _check(_get("air_qkv_rope_store")(
        qkv.data_ptr(), _DT[qkv.dtype], parts, _ptr(bias), _DT[bias.dtype] if bias is not None else 0,
        _ptr(table), rot, positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], q_out.data_ptr(), cache.data_ptr(), _DT[q_out.dtype], T, heads, kv_heads,
        head_dim, cache.shape[3], 1 if write_kv else 0, _ptr(status), _stream()), "qkv_rope_store")
    return q_out


def silu_mul(gate_up, out, block=None):
    """out[t, i] = silu(gate[t, i]) * up[t, i], where gate_up [T, 2I] holds blocks of `block` gate
    columns and `block` up columns in turn (default: all gate columns, then all up columns)."""
    T, I = out.shape
    block = I if block is None else block
    if block <= 0 or I % block:
        raise KernelError(f"silu_mul: block {block} does not divide {I}")
    _req(gate_up, "gate_up", _FLOATS, (T, 2 * I))
    _req(out, "out", _FLOATS)
    _check(_get("air_silu_mul")(gate_up.data_ptr(), _DT[gate_up.dtype], out.data_ptr(), _DT[out.dtype], T, I,
                                block, _stream()), "silu_mul")
    return out


def convert(src, out):
    _req(src, "src", _FLOATS)
    _req(out, "out", _FLOATS, tuple(src.shape))
    _check(_get("air_convert")(src.data_ptr(), _DT[src.dtype], out.data_ptr(), _DT[out.dtype], src.numel(),
                               _stream()), "convert")
    return out


def gemm_f32(a, w, bias, out):
    """out[M, N] = a[M, K] @ w[N, K]^T + bias, all float32, on the CUDA cores."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", (torch.float32,))
    _req(w, "w", (torch.float32,), (N, K))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (N,))
    _req(out, "out", (torch.float32,), (M, N))
    _check(_get("air_gemm_f32")(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, _stream()),
           "gemm_f32")
    return out


def paged_attention_ref(q, cache, block_table, token_seq, positions, out, window, scale):
    T, H, d = q.shape
    _req(q, "q", _FLOATS)
    _req(cache, "cache", (q.dtype,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (q.dtype,), (T, H, d))
    if d % 16 or d > 256:
        raise KernelError(f"head size {d}: the attention kernels take multiples of 16 up to 256")
    _check(_get("air_paged_attention_ref")(
        q.data_ptr(), cache.data_ptr(), _DT[q.dtype], block_table.data_ptr(), block_table.shape[1],
        token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(), T, H, cache.shape[2], d, cache.shape[3],
        int(window or 0), float(scale), _stream()), "paged_attention_ref")
    return out


def sample(logits, temperature, uniform, out, status=None, slots=None, last_token=None, top_k=None, top_p=None):
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or temperature is None), else the
    index drawn from softmax(logits[r] / temperature[r]) with the uniform number uniform[r], after
    keeping the top_k[r] largest logits (0: all) and of those the shortest prefix of the descending order
    that holds the share top_p[r] of the weight (1: all).  With slots and last_token, also
    last_token[slots[r]] = out[r]."""
    R, V = logits.shape
    _req(logits, "logits", (torch.float32,))
    if temperature is not None:
        _req(temperature, "temperature", (torch.float32,), (R,))
        _req(uniform, "uniform", (torch.float32,), (R,))
    if top_k is not None:
        _req(top_k, "top_k", _I32, (R,))
    if top_p is not None:
        _req(top_p, "top_p", (torch.float32,), (R,))
    _req(out, "out", _I32, (R,))
    if slots is not None:
        _req(slots, "slots", _I32, (R,))
        _req(last_token, "last_token", _I32)
    _check(_get("air_sample")(logits.data_ptr(), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
                              out.data_ptr(), _ptr(slots), _ptr(last_token), R, V, _ptr(status), _stream()), "sample")
    return out


def table_update(table, updates):
    """table[slot, block] = page for every (slot, block, page) of updates (flat int32 [3n])."""
    _req(table, "table", _I32)
    _req(updates, "updates", _I32)
    _check(_get("air_table_update")(table.data_ptr(), updates.data_ptr(), updates.numel() // 3, table.shape[1],
                                    _stream()), "table_update")
    return table


DECODE_HEAD_DIMS = (64, 128, 256)


def tile_pages(page_tokens: int) -> bool:
    """Whether the kernels that fetch 64 keys at a time with the copy engine take this page size: a tile of
    keys must lie in one page or be made of whole pages."""
    return 64 % page_tokens == 0 if page_tokens < 64 else page_tokens % 64 == 0


def decode_splits(tokens: int, heads: int, kv_heads: int) -> int:
    """How many blocks share the keys of one (token, kv head): so many that about 190 blocks run,
    which keeps every SM busy without a second round (measured on B200: 6 for 8 tokens x 4 kv heads,
    1 for 64 tokens, 32 for one token)."""
    per_split = tokens * kv_heads * (-(-(heads // kv_heads) // 16))
    return max(1, min(32, round(192 / per_split)))


def decode_attention(q, cache, block_table, token_seq, positions, out, window, scale, splits=None, scratch=None,
                     status=None, engine="tma"):
    """bfloat16 attention for one query token per request.  scratch: (float32 [T*H*splits*D], float32
    [T*H*splits*2]) or None to allocate.  engine "tma": keys and values by the copy engine into shared
    memory (attention_decode_tma.cu); "ldg": by the warps' own loads (attention_decode.cu)."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in DECODE_HEAD_DIMS:
        raise KernelError(f"decode_attention takes head sizes {DECODE_HEAD_DIMS}, not {d}")
    if splits is None:
        splits = decode_splits(T, H, K)
    po = pm = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(T * H * splits * d, dtype=torch.float32, device=q.device),
                       torch.empty(T * H * splits * 2, dtype=torch.float32, device=q.device))
        po, pm = scratch
        _req(po, "scratch[0]", (torch.float32,))
        _req(pm, "scratch[1]", (torch.float32,))
        if po.numel() < T * H * splits * d or pm.numel() < T * H * splits * 2:
            raise KernelError("decode_attention: scratch is too small")
    global launches
    if engine == "tma" and tile_pages(P):
        _check(_get("air_decode_attention_tma")(
            q.data_ptr(), cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
            token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(po), _ptr(pm), T, H, K, d, P,
            int(window or 0), float(scale), splits, _ptr(status), _stream()), "decode_attention_tma")
    else:
        _check(_get("air_decode_attention")(
            q.data_ptr(), cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], token_seq.data_ptr(),
            positions.data_ptr(), out.data_ptr(), _ptr(po), _ptr(pm), T, H, K, d, P, int(window or 0), float(scale),
            splits, _stream()), "decode_attention")
    if splits > 1:
        launches += 1
    return out


def decode_attention_fresh_ok(qkv, table, cache, head_dim) -> bool:
    """Whether decode_attention_fresh takes this: float32 product output, a table that rotates all of a head,
    pages that the copy engine's tiles fit."""
    return (qkv.dtype == torch.float32 and head_dim in DECODE_HEAD_DIMS and table is not None
            and table.shape[1] == head_dim and cache.dtype == torch.bfloat16 and tile_pages(cache.shape[3]))


def decode_attention_fresh(qkv, bias, table, cache, block_table, token_seq, positions, out, heads, window, scale,
                           write_kv=True, splits=None, status=None):
    """bfloat16 attention for one query token per request, straight from the q/k/v product: qkv float32
    [T, (H + 2K) d] or [parts, T, (H + 2K) d] partial sums; the kernel adds the bias, rotates q and k by the
    table's row of each token's position, writes k and v to the pages (write_kv) and attends, which
    qkv_rope_store followed by decode_attention do in two launches (attention_decode_tma.cu)."""
    T, H = qkv.shape[-2], heads
    d, K, P = cache.shape[4], cache.shape[2], cache.shape[3]
    width = (H + 2 * K) * d
    parts = 1 if qkv.dim() == 2 else qkv.shape[0]
    _req(qkv, "qkv", (torch.float32,), (T, width) if qkv.dim() == 2 else (parts, T, width))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (width,))
    _req(table, "table", (torch.float32,), (None, d))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if not decode_attention_fresh_ok(qkv, table, cache, d):
        raise KernelError("decode_attention_fresh: head size, rotary width or page size that this kernel does not take")
    if splits is None:
        splits = decode_splits(T, H, K)
    po = pm = None
    if splits > 1:
        po = torch.empty(T * H * splits * d, dtype=torch.float32, device=qkv.device)
        pm = torch.empty(T * H * splits * 2, dtype=torch.float32, device=qkv.device)
    _check(_get("air_decode_attention_tma_fresh")(
        qkv.data_ptr(), parts, _ptr(bias), table.data_ptr(), 1 if write_kv else 0, cache.data_ptr(), cache.shape[0],
        block_table.data_ptr(), block_table.shape[1], token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(),
        _ptr(po), _ptr(pm), T, H, K, d, P, int(window or 0), float(scale), splits, _ptr(status), _stream()),
        "decode_attention_tma")
    if splits > 1:
        global launches
        launches += 1
    return out


TILE_GROUP = 8     # the list of 16-token tiles comes in groups of 8 that belong to one request
TILE_PAIR = 16     # the tcgen05 kernel takes two groups, one after the other in a request, per block


def prefill_attention(q, cache, block_table, tiles, out, window, scale, status=None):
    """bfloat16 causal attention for tiles of up to 16 consecutive tokens of a request (see
    attention_prefill.cu).  tiles [8n, 4] int32: (slot, first token, its position, rows), in groups of
    8 tiles of one request; rows = 0 marks an empty tile."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(tiles, "tiles", _I32, (None, 4))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in DECODE_HEAD_DIMS:
        raise KernelError(f"prefill_attention takes head sizes {DECODE_HEAD_DIMS}, not {d}")
    if tiles.shape[0] % TILE_GROUP:
        raise KernelError("prefill_attention: the tile list must come in groups of 8")
    if not tile_pages(P):
        raise KernelError(f"prefill_attention: page size {P} is neither a divisor nor a multiple of 64")
    _check(_get("air_prefill_attention")(
        q.data_ptr(), cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
        tiles.data_ptr(), tiles.shape[0], out.data_ptr(), H, K, d, P, int(window or 0), float(scale), _ptr(status),
        _stream()), "prefill_attention")
    return out


EPI_F32, EPI_BF16, EPI_SILU, EPI_PARTIAL = 0, 1, 2, 3


def gemm_tc(a, w, out, bn, epi, splits=1, status=None, max_blocks=0, force_rows_as_m=False, row_ss=None, eps=0.0):
    """bfloat16 product a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (see gemm_tc.cu).
    row_ss (float32 [tiles, M]) with eps: the accumulators are multiplied per row by
    rsqrt(sum over tiles of row_ss / K + eps) before the epilogue (the kernel for few rows only; see
    add_prenorm).
    epi EPI_F32: out float32 [M,N]; EPI_BF16: out bfloat16 [M,N]; EPI_SILU: w holds gate and up rows
    interleaved in blocks of bn/2, out bfloat16 [M,N/2] = silu(gate)*up; EPI_PARTIAL: out float32
    [splits,M,N] partial sums over parts of k.  With up to 64 rows and bn 128 or 256 the product runs with the
    weights as the M side of the instruction (gemm_tc_small.cu) unless force_rows_as_m."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", (torch.bfloat16,))
    _req(w, "w", (torch.bfloat16,), (N, K))
    if K % 8:
        raise KernelError(f"gemm_tc: K = {K} must be a multiple of 8 (TMA rows are multiples of 16 bytes)")
    if bn not in (32, 64, 128, 256):
        raise KernelError(f"gemm_tc: tile width {bn}")
    if epi == EPI_F32:
        _req(out, "out", (torch.float32,), (M, N))
    elif epi == EPI_BF16:
        _req(out, "out", (torch.bfloat16,), (M, N))
    elif epi == EPI_SILU:
        _req(out, "out", (torch.bfloat16,), (M, N // 2))
        if bn < 64 or N % bn:
            raise KernelError(f"gemm_tc: silu epilogue needs N = {N} to be a multiple of the tile width {bn} >= 64")
    elif epi == EPI_PARTIAL:
        _req(out, "out", (torch.float32,), (splits, M, N))
    else:
        raise KernelError(f"gemm_tc: epilogue {epi}")
    if epi != EPI_SILU and N % 4:
        raise KernelError(f"gemm_tc: N = {N} must be a multiple of 4")
    if row_ss is not None:
        _req(row_ss, "row_ss", (torch.float32,), (None, M))
    if small_rows(M, N, bn, epi) and not force_rows_as_m:
        # few tokens: the weights are the M side of the instruction (gemm_tc_small.cu)
        _check(_get("air_gemm_tc_small")(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, bn, epi, splits,
                                         max_blocks, _ptr(status), _ptr(row_ss),
                                         0 if row_ss is None else row_ss.shape[0], float(eps), _stream()),
               "gemm_tc_small")
        return out
    if row_ss is not None:
        raise KernelError("gemm_tc: a scale per row is taken by the kernel for up to 64 rows only")
    _check(_get("air_gemm_tc")(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, bn, epi, splits, max_blocks,
                               _ptr(status), _stream()), "gemm_tc")
    return out


def small_rows(M: int, N: int, bn: int, epi: int) -> bool:
    """Whether gemm_tc takes the kernel with the weights as the M side: up to 64 tokens, tiles of 128 or
    256 rows of W; with the activation, gate and up rows in blocks of 128."""
    if M > 64 or bn not in (128, 256):
        return False
    return epi != EPI_SILU or (bn == 256 and N % 256 == 0)


TC_ATTENTION_HEAD_DIMS = (64, 128)


def prefill_attention_scratch(slots: int, head_dim: int, device):
    """Where the segments of cut items leave their partial sums: (float32 [slots, 256, d], float32 [slots, 256, 2])."""
    return (torch.empty((slots, 2 * TILE_GROUP * 16, head_dim), dtype=torch.float32, device=device),
            torch.empty((slots, 2 * TILE_GROUP * 16, 2), dtype=torch.float32, device=device))


def prefill_attention_tc(q, cache, block_table, tiles, out, window, scale, status=None, segments=None, items=None,
                         slots=0, scratch=None):
    """bfloat16 causal attention with both products on the tcgen05 tensor cores (see
    attention_prefill_tc.cu); arguments as prefill_attention; head size 64 or 128.
    segments [n, 5] int32 (pair of the list, head, first key tile, key tiles, slot or -1): which block takes which
    part of which pair's stream of keys, instead of one block per pair and head; items [m, 4] int32 (pair, head,
    first slot, slots): the (pair, head)s whose segments write partial sums into `slots` slots, merged here.
    scratch: what prefill_attention_scratch gives (or None to allocate): the layers of a step can share it."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(tiles, "tiles", _I32, (None, 4))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in TC_ATTENTION_HEAD_DIMS:
        raise KernelError(f"prefill_attention_tc takes head sizes {TC_ATTENTION_HEAD_DIMS}, not {d}")
    if tiles.shape[0] % TILE_PAIR:
        raise KernelError("prefill_attention_tc: the tile list must come in groups of 16 per request")
    if not tile_pages(P):
        raise KernelError(f"prefill_attention_tc: page size {P} is neither a divisor nor a multiple of 64")
    part_o = part_ml = None
    n_items = 0
    if segments is not None:
        _req(segments, "segments", _I32, (None, 5))
        if segments.shape[0] == 0:
            raise KernelError("prefill_attention_tc: an empty list of segments")
        if slots:
            _req(items, "items", _I32, (None, 4))
            n_items = items.shape[0]
            part_o, part_ml = scratch if scratch is not None else prefill_attention_scratch(slots, d, q.device)
            _req(part_o, "scratch[0]", (torch.float32,), (None, 2 * TILE_GROUP * 16, d))
            _req(part_ml, "scratch[1]", (torch.float32,), (None, 2 * TILE_GROUP * 16, 2))
            if part_o.shape[0] < slots or part_ml.shape[0] < slots:
                raise KernelError("prefill_attention_tc: the scratch tensors hold fewer slots than the segments name")
    _check(_get("air_prefill_attention_tc")(
        q.data_ptr(), T, cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
        tiles.data_ptr(), tiles.shape[0], _ptr(segments), 0 if segments is None else segments.shape[0],
        _ptr(items) if n_items else None, n_items, int(slots) if segments is not None else 0, _ptr(part_o), _ptr(part_ml),
        out.data_ptr(), H, K, d, P, int(window or 0), float(scale), _ptr(status), _stream()), "prefill_attention_tc")
    return out
