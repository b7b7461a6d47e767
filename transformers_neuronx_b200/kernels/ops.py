"""Python faces of the CUDA entry points: they check devices, types, shapes and strides, then pass
raw pointers and the current CUDA stream.  Nothing here computes; there is no fallback: on a tensor
that is not on a CUDA device every function raises."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from . import build as _build

_ERRORS = {-1: "bad argument", -2: "unsupported size", -3: "a bounded wait inside the kernel ran out"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """How many of this package's kernels have been launched by this process (kernels replayed
    from a CUDA graph are added by the code that replays it)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += int(n)


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_scoped_stream = None


def _stream() -> c_void_p:
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for all kernel launches inside the block (asking torch
    for it costs a few microseconds per launch, which a model step of a few tokens notices).  Enter
    it where the stream is already the one to launch on, e.g. inside a graph capture."""

    def __enter__(self):
        global _scoped_stream
        self._prev = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._prev
        return False


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None, contiguous=True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the engine has no CPU path")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {ndim}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_H16 = (torch.bfloat16, torch.float16)          # the 16-bit types: one library flavour each (kernels/build.py)
_FLOATS = (torch.float32,) + _H16

# Activations a product's epilogue applies, by the names the reference looks up
# (src/transformers_neuronx/hlo.py:485-501 -> activations.py) -> the kernels' codes (csrc/common.cuh).
ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "gelu_new": 2, "gelu_new_legacy": 2, "gelu_pytorch_tanh": 2,
               "silu": 3, "swish": 3, "sigmoid": 4, "gelu": 5}


def activation_code(name) -> int:
    if name not in ACTIVATIONS:
        raise KernelError(f"activation {name!r} is not built into the products' epilogues; "
                          f"available: {sorted(k for k in ACTIVATIONS if k)}")
    return ACTIVATIONS[name]


def _is_h16(t: torch.Tensor) -> int:
    return 1 if t.dtype in _H16 else 0


def _lib(name: str, *tensors):
    """The library `name` in the flavour of the 16-bit type among `tensors` (they must agree)."""
    kinds = {t.dtype for t in tensors if t is not None and t.dtype in _H16}
    if len(kinds) > 1:
        raise KernelError(f"{name}: bfloat16 and float16 tensors in one call")
    return _build.load(name, next(iter(kinds)) if kinds else None)


def _rows_2d(t: torch.Tensor, name: str):
    """A 2-D tensor whose rows are contiguous (a column slice of a wider buffer is allowed)."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows")
    return t.shape[0], t.shape[1], t.stride(0)


# ---------------------------------------------------------------------------------------------
def embed(tok_table, pre, ids, pos_table, positions, pos_offset, out_f32, out_act, tok_scale=1.0, sin_freq=None):
    """out[n] = tok_scale * (tok_table[ids[n]] or pre[n]) + pos_table[positions[n] + pos_offset]; with sin_freq
    (32-bit, one frequency per pair of columns) a sinusoidal vector is added as well: column 2i gets
    sin(position * sin_freq[i]), column 2i + 1 the cosine."""
    lib = _lib("embedding", tok_table, pos_table, out_act)
    N = ids.shape[0]
    _need(ids, "ids", torch.int32, 1)
    ref = out_f32 if out_f32 is not None else out_act
    H = ref.shape[1]
    table_bf16 = 0
    if tok_table is not None:
        _need(tok_table, "tok_table", _FLOATS, 2)
        if tok_table.shape[1] != H:
            raise KernelError("tok_table width differs from the output width")
        table_bf16 = _is_h16(tok_table)
    else:
        _need(pre, "pre", torch.float32, 2)
    if pos_table is not None:
        _need(pos_table, "pos_table", _FLOATS, 2)
        _need(positions, "positions", torch.int32, 1)
        if tok_table is not None and pos_table.dtype != tok_table.dtype:
            raise KernelError("token and position tables must have one dtype")
        table_bf16 = _is_h16(pos_table)
        if pos_table.shape[1] != H:
            raise KernelError("pos_table width differs from the output width")
    if out_f32 is not None:
        _need(out_f32, "out_f32", torch.float32, 2)
    act_bf16 = 0
    if out_act is not None:
        _need(out_act, "out_act", _FLOATS, 2)
        act_bf16 = _is_h16(out_act)
    if sin_freq is not None:
        _f32_vec(sin_freq, "sin_freq", (H + 1) // 2)
        _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_embed(_p(tok_table), _p(pre), _p(ids), _p(pos_table), _p(positions), c_int(pos_offset),
                         c_float(float(tok_scale)), _p(sin_freq), _p(out_f32), _p(out_act), c_int(N), c_int(H),
                         c_int(table_bf16), c_int(act_bf16), _stream()), "embed")


def patch_tokens(tokens, src, sampled):
    """tokens[i] = sampled[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
    lib = _build.load("embedding")
    for t, nm in ((tokens, "tokens"), (src, "src"), (sampled, "sampled")):
        _need(t, nm, torch.int32, 1)
    if src.shape[0] < tokens.shape[0]:
        raise KernelError("src is shorter than tokens")
    _check(lib.tnx_patch_tokens(_p(tokens), _p(src), _p(sampled), c_int(tokens.shape[0]), _stream()), "patch_tokens")


def gather_rows(table, ids, out):
    lib = _lib("embedding", table, out)
    _need(table, "table", _FLOATS, 2)
    _need(ids, "ids", torch.int32, 1)
    _need(out, "out", _FLOATS, 2)
    _check(lib.tnx_gather_rows(_p(table), _p(ids), _p(out), c_int(ids.shape[0]), c_int(table.shape[1]),
                               c_int(_is_h16(table)), c_int(_is_h16(out)), _stream()), "gather_rows")


def layer_norm(x, gamma, beta, eps, out_f32=None, out_act=None, rows=None):
    """Rows of the 32-bit x normalised; `rows` (int32) picks input rows."""
    lib = _lib("layernorm", out_act)
    _need(x, "x", torch.float32, 2)
    H = x.shape[1]
    n_rows = rows.shape[0] if rows is not None else x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    for t, nm in ((gamma, "gamma"), (beta, "beta")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != H:
                raise KernelError(f"{nm} has {t.shape[0]} elements, the rows have {H}")
    act_bf16 = 0
    for t, nm in ((out_f32, "out_f32"), (out_act, "out_act")):
        if t is not None:
            _need(t, nm, torch.float32 if nm == "out_f32" else _FLOATS, 2)
            if t.shape[0] < n_rows or t.shape[1] != H:
                raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{n_rows}, {H}]")
    if out_act is not None:
        act_bf16 = _is_h16(out_act)
    _check(lib.tnx_layer_norm(_p(x), _p(rows), _p(gamma), _p(beta), c_float(eps), _p(out_f32), _p(out_act),
                              c_int(n_rows), c_int(H), c_int(act_bf16), _stream()), "layer_norm")


def pick_rows(x, rows, out_f32=None, out_act=None):
    lib = _lib("layernorm", out_act)
    _need(x, "x", torch.float32, 2)
    n_rows = rows.shape[0] if rows is not None else x.shape[0]
    act_bf16 = _is_h16(out_act) if out_act is not None else 0
    _check(lib.tnx_pick_rows(_p(x), _p(rows), _p(out_f32), _p(out_act), c_int(n_rows), c_int(x.shape[1]),
                             c_int(act_bf16), _stream()), "pick_rows")


def gemm_simt(a, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(a @ w^T) on CUDA cores with 32-bit FMA; a [M, K], w [N, K], out [M, N]; each of
    them 32-bit or 16-bit (a 16-bit matrix is widened exactly as it is loaded)."""
    lib = _lib("gemm_simt", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _FLOATS, None, contiguous=False)
    _need(w, "w", _FLOATS, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemm_simt(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                             c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(a)),
                             c_int(_is_h16(w)), c_int(_is_h16(out)), _stream()), "gemm_simt")


def kv_append(k_src, v_src, slot_mapping, cache, page_size):
    """k_src, v_src: [N, n_kv_heads * head_dim] views (rows contiguous, one row stride);
    cache: [pages, 2, n_kv_heads, page_size, head_dim]."""
    lib = _lib("kv_cache", cache, k_src, v_src)
    _need(cache, "cache", _FLOATS, 5)
    _need(slot_mapping, "slot_mapping", torch.int32, 1)
    N, width, stride = _rows_2d(k_src, "k_src")
    if _rows_2d(v_src, "v_src") != (N, width, stride) or k_src.dtype != cache.dtype or v_src.dtype != cache.dtype:
        raise KernelError("k_src and v_src must agree in shape, stride and dtype with the cache")
    _, two, n_kv, ps, d = cache.shape
    if two != 2 or ps != page_size or n_kv * d != width:
        raise KernelError(f"cache shape {tuple(cache.shape)} does not fit rows of width {width}")
    _check(lib.tnx_kv_append(_p(k_src), _p(v_src), c_int(stride), _p(slot_mapping), _p(cache), c_int(N),
                             c_int(n_kv), c_int(d), c_int(ps), c_int(_is_h16(cache)), _stream()), "kv_append")


def copy_rows(tensor, pairs):
    """Rows (first axis) of a contiguous tensor copied within it: for each (source, destination) of the
    int32 tensor `pairs` [n, 2], row destination takes the contents of row source.  No row may be both."""
    lib = _build.load("kv_cache")
    if not tensor.is_cuda or not tensor.is_contiguous() or tensor.dim() < 1:
        raise KernelError("copy_rows needs a contiguous tensor on the GPU")
    _need(pairs, "pairs", torch.int32, 2)
    if pairs.shape[1] != 2:
        raise KernelError("pairs must be [n, 2]")
    row_bytes = tensor[0].numel() * tensor.element_size() if tensor.shape[0] else 0
    _check(lib.tnx_copy_rows(_p(tensor), _p(pairs), c_int(pairs.shape[0]), ctypes.c_longlong(row_bytes), _stream()), "copy_rows")


def mask_rule(window=0, chunk=0) -> int:
    """Which earlier keys a query reads, as the one number the attention kernels take (csrc/common.cuh:
    first_visible_key): 0 all of them, w > 0 the last w (sliding window), -c those of the query's own block of c
    positions, blocks counted from position 0 of the sequence (chunked mask)."""
    window, chunk = int(window or 0), int(chunk or 0)
    if window < 0 or chunk < 0:
        raise KernelError("a window and a chunk are positive numbers of positions (0: none)")
    if window and chunk:
        raise KernelError("the attention kernels take a sliding window or a chunked mask, not both")
    return -chunk if chunk else window


def attention_simt(q, cache, block_tables, token_request, positions, out, n_heads, scale, window=0, chunk=0):
    """q: [N, n_heads * head_dim] view; out likewise; cache as in kv_append."""
    lib = _lib("attention_simt", cache, q, out)
    _need(cache, "cache", _FLOATS, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_attention_simt(_p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
                                  _p(token_request), _p(positions), _p(out), c_int(out_stride), c_int(N),
                                  c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(mask_rule(window, chunk)),
                                  c_float(scale), c_int(_is_h16(cache)), _stream()), "attention_simt")


def sample(logits, out, temperature=None, top_k=None, top_p=None, seeds=None, counters=None, suppress_id=-1,
           min_keep=None, deterministic=False):
    """out[r] = next token of row r; per-row float32 temperature (<= 0: greedy), int32 top_k
    (0: off), float32 top_p (1: off), int32 min_keep (the fewest tokens top-p keeps; None: 1), int64
    seeds and counters for the Philox draw.  deterministic: no draw; the kept tokens are taken from
    the most likely down and the first at which the summed probability reaches one half is chosen."""
    lib = _build.load("sampling")
    _need(logits, "logits", torch.float32, None, contiguous=False)
    R, V, ld = _rows_2d(logits, "logits")
    _need(out, "out", torch.int32, 1)
    for t, nm, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                      (top_p, "top_p", torch.float32), (min_keep, "min_keep", torch.int32),
                      (seeds, "seeds", torch.int64), (counters, "counters", torch.int64)):
        if t is not None:
            _need(t, nm, dt, 1)
            if t.shape[0] < R:
                raise KernelError(f"{nm} has fewer entries than there are rows")
    _check(lib.tnx_sample(_p(logits), c_int(ld), c_int(R), c_int(V), _p(temperature), _p(top_k), _p(top_p),
                          _p(min_keep), c_int(1 if deterministic else 0), _p(seeds), _p(counters),
                          c_int(suppress_id), _p(out), _stream()), "sample")


def sample_packed(logits, packed, with_top_p, out, err_word=None):
    """sample() with every row's parameters packed, 16 int32 words a row (csrc/sampling.cu):
    temperature, top_k, top_p, min_keep, seed (2), counter (2), flags, up to four suppressed ids.
    err_word: a device int32 whose value is written to out[rows] (out then needs rows + 1 entries)."""
    lib = _build.load("sampling")
    _need(logits, "logits", torch.float32, None, contiguous=False)
    R, V, ld = _rows_2d(logits, "logits")
    _need(out, "out", torch.int32, 1)
    _need(packed, "packed", torch.int32, None)
    words = lib.tnx_sample_row_words()
    if packed.numel() < R * words:
        raise KernelError(f"packed holds {packed.numel()} words, {R} rows need {R * words}")
    if out.shape[0] < R + (1 if err_word is not None else 0):
        raise KernelError("out is too short for the rows (and the error word)")
    if err_word is not None:
        _need(err_word, "err_word", torch.int32, 1)
    _check(lib.tnx_sample_packed(_p(logits), c_int(ld), c_int(R), c_int(V), _p(packed), c_int(1 if with_top_p else 0),
                                 _p(err_word), _p(out), _stream()), "sample")


def sample_force_blocks_per_row(blocks=None) -> None:
    """The sampling kernel with 1, 2, 4 or 8 thread blocks a row whatever the sizes (None: its own rule
    again).  For the test that draws the same tokens with each; not for serving."""
    _check(_build.load("sampling").tnx_sample_force_blocks_per_row(c_int(int(blocks or 0))), "sample_force_blocks_per_row")


def error_word(device) -> torch.Tensor:
    """The device word that kernels with bounded waits set when a wait ran out (0: none did)."""
    return _state(device)["err"]


def raise_if_error_code(code: int, where: str = "") -> None:
    """Raises for a value of the error word that was read along with a step's results."""
    if code:
        for st in _dev_state.values():
            st["err"].zero_()
        raise KernelError(f"a bounded wait ran out inside a kernel{where} (where: {code}); its results, and "
                          "everything computed from them, are invalid")


# ---------------------------------------------------------------------------------------------
# Tensor-core kernels (bfloat16).
_attention_impls = {}
_gemm_plans = {}          # (M, N, K, SMs) -> (splits, scratch bytes, counters) as the library plans them
_dev_state = {}          # per device: error word, split-K scratch and counters, SM count


def _state(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _dev_state.get(key)
    if st is None:
        st = {"err": torch.zeros(1, dtype=torch.int32, device=device),
              "scratch": None, "counters": torch.zeros(1024, dtype=torch.int32, device=device),
              "sms": torch.cuda.get_device_properties(device).multi_processor_count}
        _dev_state[key] = st
    return st


def _grow(st, key, need, dtype, device, minimum, zero=False):
    """Scratch buffer `key` with at least `need` elements.  A buffer that is outgrown is kept alive:
    captured CUDA graphs still hold its address."""
    cur = st.get(key)
    if cur is None or cur.numel() < need:
        if cur is not None:
            st.setdefault("retired", []).append(cur)
        n = max(int(need), int(minimum))
        st[key] = torch.zeros(n, dtype=dtype, device=device) if zero else torch.empty(n, dtype=dtype, device=device)
    return st[key]


def raise_on_device_error(device=None):
    """Reads the error word that kernels with bounded waits set (this synchronises)."""
    for key, st in _dev_state.items():
        code = int(st["err"].item())
        if code:
            st["err"].zero_()
            raise KernelError(f"a bounded wait ran out inside a kernel on cuda:{key} (where: {code}); "
                              "its results are invalid")


def selftest_wait_runs_out(device, code: int = 99, limit_ns: int = 1_000_000) -> None:
    """Launches a kernel whose bounded wait (about a millisecond) runs out by design and records
    `code` in the device's error word: what raise_on_device_error() and the engine's per-step check
    then report.  For tests of the error path; nothing hangs, the wait ends by itself."""
    lib = _build.load("gemm_tc")
    st = _state(torch.device(device))
    _check(lib.tnx_selftest_wait_runs_out(_p(st["err"]), c_int(code), ctypes.c_longlong(limit_ns), _stream()),
           "selftest_wait_runs_out")


def gemm_tc_supported(a, w, out) -> bool:
    """Size rules of the TMA descriptors: row pitches multiples of 16 bytes, 16-byte aligned bases."""
    if a.dtype not in _H16 or w.dtype != a.dtype or (out.dtype in _H16 and out.dtype != a.dtype):
        return False
    K = a.shape[1]
    if K % 8 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return False
    return out.data_ptr() % 16 == 0


def gemv(a, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(a @ w^T) for one to four tokens, the weights streamed through the multiply-add
    units (16-bit operands, 32-bit sums).  gemm_tc() picks it by itself for one token."""
    lib = _lib("gemv", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _H16, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemv shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not lib.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)) or not gemm_tc_supported(a, w, out):
        raise KernelError("gemv takes one to four tokens, K a multiple of 8 and 16-byte aligned rows")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemv(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                        c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                        _stream()), "gemv")


def gemv_layer_norm_supported(x, w, out) -> bool:
    """Whether gemv_layer_norm takes these tensors: one token (measured on the 6.7B sizes: a decode step of one
    request 3.15 -> 3.11 ms; with two requests the tensor-core product after a LayerNorm kernel takes 3.40 ms
    and this kernel 3.90), 32-bit rows of x, a 16-bit matrix, 16-byte aligned rows, the row within shared memory."""
    if x.dim() != 2 or x.dtype != torch.float32 or w.dtype not in _H16 or x.shape[0] != 1:
        return False
    if out.dtype in _H16 and out.dtype != w.dtype:
        return False
    K = x.shape[1]
    return (w.dim() == 2 and w.shape[1] == K and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 4 == 0
            and x.data_ptr() % 16 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and K * 6 <= 112 * 1024)


def gemv_layer_norm(x, gamma, beta, eps, w, out, bias=None, residual=None, activation=None):
    """out = epilogue(LayerNorm(x) @ w^T) for one to four tokens: x are 32-bit rows (the residual stream),
    normalized in 32-bit by every thread block of the product as it stages its activations, rounded to
    the matrix's 16-bit type as a LayerNorm kernel would round them."""
    lib = _lib("gemv", w, out)
    act = activation_code(activation)
    _need(x, "x", torch.float32, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, ldx = _rows_2d(x, "x")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemv shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not lib.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)):
        raise KernelError("gemv takes one to four tokens and K a multiple of 8")
    for t, nm in ((gamma, "gamma"), (beta, "beta")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.shape[0] != K:
                raise KernelError(f"{nm} length differs from the row length")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    _check(lib.tnx_gemv_ln(_p(x), c_int(ldx), _p(gamma), _p(beta), c_float(float(eps)), _p(w), _p(bias), _p(residual), _p(out),
                           c_int(M), c_int(N), c_int(K), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                           _stream()), "gemv_layer_norm")


def gemm_tc(a, w, out, bias=None, residual=None, activation=None, splits=None, few_tokens_kernel=True, cluster=False):
    """out = epilogue(a @ w^T), 16-bit operands (both bfloat16 or both float16), 32-bit accumulation: on the tcgen05 tensor cores,
    or (one token, unless few_tokens_kernel is False or splits is given) as a stream of the
    weights through the multiply-add units.  `splits` forces a split of K for up to 128 tokens (a test
    hook): partial tiles added by the CTA that finishes last, or (cluster=True, at most 8 splits) by
    the CTAs of a cluster through their shared memory, which is what the kernel's own plan uses."""
    lib = _lib("gemm_tc", a, w, out)
    act = activation_code(activation)
    _need(a, "a", _H16, None, contiguous=False)
    _need(w, "w", _H16, None, contiguous=False)
    _need(out, "out", _FLOATS, None, contiguous=False)
    M, K, lda = _rows_2d(a, "a")
    N, Kw, ldw = _rows_2d(w, "w")
    Mo, No, ldc = _rows_2d(out, "out")
    if Kw != K or Mo != M or No != N:
        raise KernelError(f"gemm shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not gemm_tc_supported(a, w, out):
        raise KernelError("the tensor-core product needs K and the row pitches to be multiples of 8 elements "
                          "and 16-byte aligned bases; use gemm_simt for other sizes")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != N:
            raise KernelError("bias length differs from the output width")
    if residual is not None:
        _need(residual, "residual", torch.float32, None, contiguous=False)
        if tuple(residual.shape) != (M, N) or _rows_2d(residual, "residual")[2] != ldc or out.dtype != torch.float32:
            raise KernelError("residual must be float32 with the shape and row stride of a float32 out")
    if few_tokens_kernel and splits is None and M == 1:    # with two tokens and more the tensor-core kernel is as fast (measured)
        gv = _lib("gemv", a, w, out)
        if gv.tnx_gemv_supported(c_int(M), c_int(N), c_int(K)):
            _check(gv.tnx_gemv(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                               c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                               _stream()), "gemv")
            return
    st = _state(a.device)
    plan = _gemm_plans.get((M, N, K, st["sms"]))
    if plan is None:
        n_splits, nbytes, ncnt = c_int(1), ctypes.c_longlong(0), c_int(0)
        lib.tnx_gemm_tc_plan(c_int(M), c_int(N), c_int(K), c_int(st["sms"]), ctypes.byref(n_splits),
                             ctypes.byref(nbytes), ctypes.byref(ncnt))
        if len(_gemm_plans) > 4096:
            _gemm_plans.clear()
        plan = _gemm_plans[(M, N, K, st["sms"])] = (n_splits.value, nbytes.value, ncnt.value)
    n_splits, nbytes, ncnt = c_int(plan[0]), ctypes.c_longlong(plan[1]), c_int(plan[2])
    if splits is not None and M <= lib.tnx_gemm_tc_few_tokens():
        kb = -(-K // 64)
        s = max(1, min(int(splits), kb))
        per = -(-kb // s)
        s = -(-kb // per)
        bn = 16 if M <= 16 else (32 if M <= 32 else (64 if M <= 64 else 128))
        tiles = -(-N // 128)
        n_splits, nbytes, ncnt = c_int(s), ctypes.c_longlong(s * tiles * 128 * bn * 4 if s > 1 else 0), c_int(tiles if s > 1 else 0)
        if cluster:
            if s > 8:
                raise KernelError("a cluster holds at most 8 thread blocks")
            nbytes, ncnt = ctypes.c_longlong(0), c_int(0)
    scratch = None
    if nbytes.value:
        need = nbytes.value // 4
        scratch = _grow(st, "scratch", need, torch.float32, a.device, 1 << 22)
        _grow(st, "counters", ncnt.value, torch.int32, a.device, 1024, zero=True)
    _check(lib.tnx_gemm_tc(_p(a), _p(w), _p(bias), _p(residual), _p(out), c_int(M), c_int(N), c_int(K),
                           c_int(lda), c_int(ldw), c_int(ldc), c_int(act), c_int(_is_h16(out)),
                           n_splits, _p(scratch), _p(st["counters"]), _p(st["err"]), _stream()), "gemm_tc")


GEMM_PLANS = {"tiles_128": 0, "pairs": 1, "persistent": 2, "pairs_shared": 4,
              "split_1": 31, "split_2": 32, "split_4": 34, "split_8": 38}


def gemm_tc_force_plan(plan=None, dtype=torch.bfloat16) -> None:
    """Imposes one kernel on every tensor-core product of more than 128 tokens (None: the library's
    own estimates choose again).  A product whose sizes do not allow the plan is refused.  For the
    test that times every candidate against the estimates' choice; not for serving."""
    lib = _build.load("gemm_tc", dtype)
    lib.tnx_gemm_tc_force_plan(c_int(-1 if plan is None else GEMM_PLANS[plan]))
    _gemm_plans.clear()


def decode_attention_plan(pairs: int, sms: int, head_dim: int, max_pages: int):
    """(warps a block, splits of the context) for `pairs` (row, head) pairs of decode attention.

    An SM holds sixteen warps of this kernel: four blocks of four, two of eight or one of sixteen.
    Measured at 1 to 64 rows of 32, 40 and 56 heads of 128 dims over contexts of 2,040 (every plan
    against the one chosen here), the fastest plan keeps all blocks on the GPU at once where it can and
    gives the SMs equal numbers of them:
      * few pairs: blocks of eight warps, as many splits as fill two blocks per SM (1 / 2 rows of 32
        heads: 13 / 18 us);
      * about one pair per SM (0.75 to 1): one block of sixteen warps each and no split (4 rows: 28 us,
        eight warps and two splits 30);
      * up to a third of four blocks per SM: four warps and three splits (6 rows: 39 us; eight warps and
        no split, which leaves the SMs one or two blocks each, 47);
      * up to two pairs per SM: eight warps, no split (8 rows: 49 us);
      * up to 2.7 pairs per SM: four warps and three splits again (12 rows: 73 us; without splits the SMs
        hold two or three blocks each, 80);
      * up to four pairs per SM: four warps, no split (16 rows: 91 us); beyond: four or eight warps, whichever
        an estimate of waves x (streaming + cost of a block) makes the faster (64 rows: eight warps, 321 us;
        256 rows over 256 tokens: four warps, 176 against 208 us).
    (kernels/microbench.py attention-plans repeats the sweep.)  A split keeps at least eight pages, and contexts of fewer than 48 pages are not split in three (at
    500 tokens the plans without splits were 7-12 % faster there, and from a quarter of a pair per SM
    one block of sixteen warps was: 9 against 12 us at 3 rows)."""
    most = max(1, max_pages // 8)
    wide = 16 if head_dim <= 128 else 8
    if pairs * 4 <= sms * 3:
        if most <= 4 and pairs * 4 >= sms:
            return wide, 1
        return 8, max(1, min(most, 32, (2 * sms) // max(1, pairs)))
    if pairs <= sms:
        return wide, 1
    if pairs * 3 <= 4 * sms and most >= 6:
        return 4, 3
    if pairs <= 2 * sms:
        return 8, 1
    if pairs * 10 <= sms * 27 and most >= 6:
        return 4, 3
    if pairs <= 4 * sms:
        return 4, 1
    # More pairs than the GPU holds blocks: blocks of four warps (four an SM) or of eight (two an SM) follow
    # one another.  A block costs 0.6 / 2.2 us beside its pages' streaming (8,192 pairs over 256 tokens: 176
    # against 208 us), and the last wave of blocks is as long as a full one (1,280 pairs over 1,024 tokens:
    # 123 us in three waves of four-warp blocks, 115 us in five of eight-warp ones; over 256 tokens 37 against 41).
    page_us = 16 * head_dim * 4 / 6.5e6                      # one page of keys and values at 6.5 TB/s
    t4 = -(-pairs // (4 * sms)) * (4 * sms * max_pages * page_us + 0.6)
    t8 = -(-pairs // (2 * sms)) * (2 * sms * max_pages * page_us + 2.2)
    return (4, 1) if t4 < t8 else (8, 1)


def attention_decode(q, cache, block_tables, token_request, positions, out, n_heads, scale, window=0, rows=None,
                     n_rows=None, max_kv_len=None, n_splits=None, new_kv=None, warps=None, grouped=None, chunk=0):
    """One query token per row over the paged 16-bit cache.  `rows` (int32) names the rows of q
    that are decode tokens (None: all); max_kv_len bounds their contexts (for the split plan).
    new_kv = (k, v), [rows of q, kv_heads * head_dim] bfloat16: the keys and values of the rows' own
    tokens, which the kernel then writes into their pages itself (no kv_append before it).
    n_splits (with warps, 4 or 8 a block) forces a plan: a test hook.  grouped: with 2 or 4 query heads a key/value
    head a block can take all query heads of a key/value head and read the head's pages once (None: where that pays;
    True / False: a test hook)."""
    lib = _lib("attention_decode", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    _need(block_tables, "block_tables", torch.int32, 2)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    R = int(n_rows) if n_rows is not None else (rows.shape[0] if rows is not None else N)
    st = _state(q.device)
    max_pages = max(1, -(-(int(max_kv_len) if max_kv_len is not None else block_tables.shape[1] * ps) // ps))
    forced_warps, warps = warps, 4
    # with grouped key/value heads (2 or 4 query heads each) a block takes all query heads of a key/value head
    # Measured (32 query heads of 128 on 8 key/value heads, contexts of 2,048): the grouped form wins from 64 rows on
    # (a layer's step 1.58 against 1.77 ms at 64 rows, 2.44 against 2.78 at 128) and loses below (1.34 against 1.18 at 32:
    # its blocks are a quarter as many, one an SM), so it runs once the (row, key/value head) pairs are three an SM.
    heads_per_block = lib.tnx_attention_decode_heads_per_block(c_int(n_heads), c_int(n_kv), c_int(d))
    # Measured again with 8 query heads a key/value head (the two maps of differential attention; 64 heads on 8, contexts
    # of 2,048): between two thirds of a block and three blocks an SM the grouped form wins as well when its blocks are
    # four warps and the context is split so that about two blocks an SM run (8 rows: 75 us with two splits against 93
    # with a block a head; 16 rows: 123 against 153; the plan drawn for one head a block gave 107 and 206 there).
    few_grouped = False
    if heads_per_block > 1 and grouped is None:
        blocks = R * n_heads // heads_per_block
        if blocks < 3 * st["sms"]:
            few_grouped = 3 * blocks >= 2 * st["sms"] and n_splits is None
            if not few_grouped:
                heads_per_block = 1
    elif grouped is False:
        heads_per_block = 1
    if few_grouped:
        warps = 4
        n_splits = max(1, min(max_pages // 8, (2 * st["sms"] + blocks // 2) // blocks))
        pps = -(-max_pages // n_splits)
        pps = -(-pps // warps) * warps
    elif n_splits is None:
        warps, n_splits = decode_attention_plan(R * n_heads // heads_per_block, st["sms"], d, max_pages)
        if heads_per_block > 1 and warps == 16:
            warps = 8                                           # their accumulators leave no registers for sixteen warps
        pps = -(-max_pages // n_splits)
        pps = -(-pps // warps) * warps
    else:                                                  # a test's own plan (warps: 4, 8 or 16 a block)
        warps = int(forced_warps or 4)
        n_splits = max(1, min(int(n_splits), max_pages))
        pps = -(-max_pages // n_splits)
    n_splits = -(-max_pages // pps)
    scratch = None
    if n_splits > 1:
        need = R * n_heads * n_splits * (d + 2)
        scratch = _grow(st, "att_scratch", need, torch.float32, q.device, 1 << 20)
        _grow(st, "att_counters", R * n_heads, torch.int32, q.device, 8192, zero=True)
    k_new = v_new = None
    kv_stride = 0
    if new_kv is not None:
        k_new, v_new = new_kv
        for t, nm in ((k_new, "k"), (v_new, "v")):
            _need(t, nm, cache.dtype, None, contiguous=False)
            if _rows_2d(t, nm)[:2] != (N, n_kv * d):
                raise KernelError(f"new {nm} must be [{N}, {n_kv * d}]")
        kv_stride = k_new.stride(0)
        if v_new.stride(0) != kv_stride:
            raise KernelError("new k and v must have the same row pitch")
    _check(lib.tnx_attention_decode_append(
        _p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
        _p(rows), _p(token_request), _p(positions), _p(out), c_int(out_stride), c_int(R),
        c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(mask_rule(window, chunk)), c_float(scale),
        c_int(n_splits), c_int(pps), _p(scratch), _p(st.get("att_counters")), _p(k_new), _p(v_new), c_int(kv_stride),
        c_int(warps), c_int(heads_per_block), _stream()), "attention_decode")


ATTN_PREFILL_TILE = 128      # query rows of one work item of the prefill attention kernel


def attention_prefill(q, cache, block_tables, tile_req, tile_q0, q_start, q_len, ctx_len, out, n_heads, scale,
                      window=0, n_items=None, chunk=0):
    """Causal attention of prompt portions: work items (request, first row of an ATTN_PREFILL_TILE-row tile)."""
    lib = _lib("attention_prefill", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    _, _, n_kv, ps, d = cache.shape
    if width != n_heads * d or (No, wo) != (N, width) or q.dtype != cache.dtype or out.dtype != cache.dtype:
        raise KernelError("q/out do not fit the cache's head size or dtype")
    for t, nm in ((block_tables, "block_tables"), (tile_req, "tile_req"), (tile_q0, "tile_q0"), (q_start, "q_start"),
                  (q_len, "q_len"), (ctx_len, "ctx_len")):
        _need(t, nm, torch.int32, 2 if nm == "block_tables" else 1)
    n = int(n_items) if n_items is not None else tile_req.shape[0]
    _check(lib.tnx_attention_prefill(_p(q), c_int(q_stride), _p(cache), _p(block_tables), c_int(block_tables.stride(0)),
                                     _p(tile_req), _p(tile_q0), _p(q_start), _p(q_len), _p(ctx_len), _p(out),
                                     c_int(out_stride), c_int(n), c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps),
                                     c_int(mask_rule(window, chunk)), c_float(scale), _stream()), "attention_prefill")


def attention_prefill_tc_supported(q, cache, out) -> bool:
    """The tcgen05 prefill kernel takes head sizes 64, 80, 96, 112 and 128, pages of 16 and 16-byte aligned rows."""
    return (cache.dtype in _H16 and q.dtype == cache.dtype and out.dtype == cache.dtype and cache.shape[4] in (64, 80, 96, 112, 128) and cache.shape[3] == 16 and q.stride(0) % 8 == 0 and
            out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and
            cache.shape[0] * 2 * cache.shape[2] * 16 < 2 ** 31)


def attention_prefill_tc(q, cache, block_tables, tile_req, tile_q0, q_start, q_len, ctx_len, out, n_heads, scale,
                         window=0, n_items=None, chunk=0):
    """attention_prefill on the tcgen05 tensor cores (head sizes 64 to 128 in steps of 16).  The cache must hold finite
    numbers in every row, written or not (CacheStorage allocates it zeroed)."""
    lib = _lib("attention_prefill_tc", cache, q, out)
    _need(cache, "cache", _H16, 5)
    N, width, q_stride = _rows_2d(q, "q")
    No, wo, out_stride = _rows_2d(out, "out")
    n_pages, _, n_kv, ps, d = cache.shape
    if not attention_prefill_tc_supported(q, cache, out) or width != n_heads * d or (No, wo) != (N, width):
        raise KernelError("attention_prefill_tc takes a 16-bit type, head sizes 64 to 128 in steps of 16, pages of 16, 16-byte aligned rows")
    for t, nm in ((block_tables, "block_tables"), (tile_req, "tile_req"), (tile_q0, "tile_q0"), (q_start, "q_start"),
                  (q_len, "q_len"), (ctx_len, "ctx_len")):
        _need(t, nm, torch.int32, 2 if nm == "block_tables" else 1)
    n = int(n_items) if n_items is not None else tile_req.shape[0]
    st = _state(q.device)
    _check(lib.tnx_attention_prefill_tc(_p(q), c_int(q_stride), c_int(N), _p(cache), ctypes.c_longlong(n_pages * 2 * n_kv * ps),
                                        _p(block_tables), c_int(block_tables.stride(0)), _p(tile_req), _p(tile_q0),
                                        _p(q_start), _p(q_len), _p(ctx_len), _p(out), c_int(out_stride), c_int(n),
                                        c_int(n_heads), c_int(n_kv), c_int(d), c_int(ps), c_int(mask_rule(window, chunk)),
                                        c_float(scale), _p(st["err"]), _stream()), "attention_prefill_tc")


def _attention_h16(ctx, group, q, cache, out, n_heads, scale, window, new_kv, chunk=0):
    if cache.shape[3] != 16 or cache.shape[4] > 256 or q.stride(0) % 8 or q.data_ptr() % 16:
        return False                             # rows wider than 256 dims: the CUDA-core kernel takes up to 768
    bt = ctx.block_tables[group]
    fused = None
    if new_kv is not None:
        k, v, slots = new_kv
        if ctx.decode_only and not ctx.n_prefill_tiles and k.stride(0) % 8 == 0 and k.data_ptr() % 16 == 0 \
                and v.data_ptr() % 16 == 0:
            fused = (k, v)                       # a decode step: the attention kernel appends by itself
        else:
            kv_append(k, v, slots, cache, ctx.page_size)
    if ctx.n_prefill_tiles:
        prefill = attention_prefill_tc if attention_prefill_tc_supported(q, cache, out) else attention_prefill
        prefill(q, cache, bt, ctx.tile_req, ctx.tile_q0, ctx.q_start, ctx.q_len, ctx.ctx_len, out,
                n_heads, scale, window, n_items=ctx.n_prefill_tiles, chunk=chunk)
    if ctx.n_decode_rows:
        attention_decode(q, cache, bt, ctx.token_request, ctx.positions, out, n_heads, scale, window,
                         rows=None if ctx.decode_only else ctx.decode_rows, n_rows=ctx.n_decode_rows,
                         max_kv_len=ctx.max_decode_ctx, new_kv=fused, chunk=chunk)
    return True


_attention_impls["h16"] = _attention_h16


def attention(ctx, group, q, cache, out, n_heads, scale, window=0, new_kv=None, chunk=0):
    """Attention of this step's queries over the cache of the running schedule entry.  32-bit
    caches, and head sizes or windows that the 16-bit kernels do not take, run on the CUDA-core
    kernel; a 16-bit cache runs the prefill kernel for requests with several rows and the split
    decode kernel for requests with one.  new_kv = (k, v, slot_mapping): the keys and values of
    this step's tokens, not yet in the cache; they are appended here, by kv_append or (a step of
    decode tokens only, 16-bit) by the decode kernel itself; None: the cache holds them already (a mixer that
    reads another mixer's pages).  window / chunk: see mask_rule."""
    impl = _attention_impls.get("h16") if cache.dtype in _H16 else None
    if impl is not None and impl(ctx, group, q, cache, out, n_heads, scale, window, new_kv, chunk):
        return
    if new_kv is not None:
        kv_append(new_kv[0], new_kv[1], new_kv[2], cache, ctx.page_size)
    attention_simt(q, cache, ctx.block_tables[group], ctx.token_request, ctx.positions, out, n_heads, scale,
                   window, chunk)


# ---------------------------------------------------------------------------------------------
# RMS norm, rotations by position, recurrent mixers, the gated feed-forward's elementwise step.
def _f32_vec(t, name, n=None):
    if t is None:
        return
    _need(t, name, torch.float32, 1)
    if n is not None and t.shape[0] != n:
        raise KernelError(f"{name} has {t.shape[0]} elements, expected {n}")


def rms_norm(x, weight, eps, out_f32=None, out_act=None, rows=None, x_scale=1.0, delta=None, weight_offset=0.0,
             out_scale=1.0):
    """Rows of y = x_scale * x + delta (delta optional, 32-bit like x) divided by their root mean square
    (eps inside the root) and multiplied by (weight + weight_offset) when a weight is given, then by out_scale.
    out_f32 may be x itself.  `rows` (int32) picks input rows."""
    lib = _lib("rmsnorm", out_act)
    _need(x, "x", torch.float32, 2)
    H = x.shape[1]
    n_rows = rows.shape[0] if rows is not None else x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if tuple(delta.shape) != tuple(x.shape):
            raise KernelError("delta must have the shape of x")
    _f32_vec(weight, "weight", H)
    for t, nm in ((out_f32, "out_f32"), (out_act, "out_act")):
        if t is not None:
            _need(t, nm, torch.float32 if nm == "out_f32" else _FLOATS, 2)
            if t.shape[0] < n_rows or t.shape[1] != H:
                raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{n_rows}, {H}]")
    _check(lib.tnx_rms_norm(_p(x), c_float(x_scale), _p(delta), _p(rows), _p(weight), c_float(weight_offset),
                            c_float(eps), c_float(out_scale), _p(out_f32), _p(out_act), c_int(n_rows), c_int(H),
                            c_int(_is_h16(out_act) if out_act is not None else 0), _stream()), "rms_norm")


def rms_norm_pair(x, weight1, offset1, eps1, out1, weight2=None, offset2=0.0, eps2=0.0, out2=None):
    """Two RMS norms of the same rows of the 32-bit x with one pass over them (the inputs of two sublayers that read the
    same stream): out_i = x / sqrt(mean(x^2) + eps_i) * (weight_i + offset_i), in the activation type.  out2 None: one."""
    lib = _lib("rmsnorm", out1, out2)
    _need(x, "x", torch.float32, 2)
    N, H = x.shape
    _f32_vec(weight1, "weight1", H); _f32_vec(weight2, "weight2", H)
    for t, nm in ((out1, "out1"), (out2, "out2")):
        if t is not None:
            _need(t, nm, out1.dtype if nm == "out2" else _FLOATS, 2)
            if tuple(t.shape) != (N, H):
                raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{N}, {H}]")
    _check(lib.tnx_rms_norm_pair(_p(x), _p(weight1), c_float(offset1), c_float(eps1), _p(weight2), c_float(offset2),
                                 c_float(eps2), _p(out1), _p(out2), c_int(N), c_int(H), c_int(_is_h16(out1)), _stream()),
           "rms_norm_pair")


def scaled_residual_add(x, a, scale_a=None, b=None, scale_b=None, then=None):
    """x += scale_a * a (+ scale_b * b), all 32-bit; the scales are vectors over the hidden axis (None: 1).
    then = (weight1, offset1, eps1, out1, weight2, offset2, eps2, out2): the new rows' two RMS norms (as rms_norm_pair
    forms them; out2 None: one) are written in the same kernel: the inputs of the sublayers of the layer that follows."""
    out1 = then[3] if then is not None else None
    out2 = then[7] if then is not None else None
    lib = _lib("rmsnorm", out1, out2)
    _need(x, "x", torch.float32, 2)
    N, H = x.shape
    for t, nm in ((a, "a"), (b, "b")):
        if t is not None:
            _need(t, nm, torch.float32, 2)
            if tuple(t.shape) != (N, H):
                raise KernelError(f"{nm} must have the shape of x")
    _f32_vec(scale_a, "scale_a", H); _f32_vec(scale_b, "scale_b", H)
    w1 = w2 = None
    off1 = eps1 = off2 = eps2 = 0.0
    if then is not None:
        w1, off1, eps1, _, w2, off2, eps2, _ = then
        _f32_vec(w1, "weight1", H); _f32_vec(w2, "weight2", H)
        for t, nm in ((out1, "out1"), (out2, "out2")):
            if t is not None:
                _need(t, nm, out1.dtype if nm == "out2" else _FLOATS, 2)
                if tuple(t.shape) != (N, H):
                    raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{N}, {H}]")
    _check(lib.tnx_scaled_residual_add(_p(x), _p(a), _p(scale_a), _p(b), _p(scale_b), c_int(N), c_int(H), _p(w1),
                                       c_float(off1), c_float(eps1), _p(out1), _p(w2), c_float(off2), c_float(eps2), _p(out2),
                                       c_int(_is_h16(out1) if out1 is not None else 0), _stream()), "scaled_residual_add")


def rms_norm_add(x, add_scale, delta, weight, eps, out_f32=None, out_act=None, weight_offset=0.0, then=None):
    """x + add_scale * (delta / rms(delta) * (weight + weight_offset)): the norm on a sublayer's output alone, added to
    the 32-bit stream x.  out_f32 may be x itself.  then = (weight or None, weight_offset, eps): out_act receives that
    further RMS norm of the new row (the input of the sublayer that follows) instead of the row's copy."""
    lib = _lib("rmsnorm", out_act)
    _need(x, "x", torch.float32, 2)
    _need(delta, "delta", torch.float32, 2)
    if tuple(delta.shape) != tuple(x.shape):
        raise KernelError("delta must have the shape of x")
    N, H = x.shape
    _f32_vec(weight, "weight", H)
    for t, nm in ((out_f32, "out_f32"), (out_act, "out_act")):
        if t is not None:
            _need(t, nm, torch.float32 if nm == "out_f32" else _FLOATS, 2)
            if tuple(t.shape) != (N, H):
                raise KernelError(f"{nm} has shape {tuple(t.shape)}, needs [{N}, {H}]")
    w_then, off_then, eps_then = then if then is not None else (None, 0.0, 0.0)
    _f32_vec(w_then, "the following norm's weight", H)
    _check(lib.tnx_rms_norm_add(_p(x), c_float(add_scale), _p(delta), _p(weight), c_float(weight_offset), c_float(eps),
                                _p(out_f32), _p(out_act), c_int(N), c_int(H),
                                c_int(_is_h16(out_act) if out_act is not None else 0), c_int(1 if then is not None else 0),
                                _p(w_then), c_float(off_then), c_float(eps_then), _stream()), "rms_norm_add")


def conv_qkv_prep(proj, col0, conv_w, taps, state, ctx, q_norm, k_norm, eps, inv_freq, rot_dims, interleaved, magnitude,
                  q_out, k_out, v_out, n_heads, n_kv_heads, k_dim, v_dim, pad_dim):
    """From one product's output `proj` [N, *] (from column col0 on: queries, then keys and values unless n_kv_heads is
    0): each channel's short causal convolution over the request's positions (conv_w [channels, taps] 32-bit; None:
    none), whose past comes from this step's rows or from `state` [slots, taps - 1, channels] (brought up to date here);
    queries and keys normalised per head (q_norm, k_norm [k_dim]; None: not), then turned by position on their first
    rot_dims dims (interleaved pairs or halves; sines and cosines times `magnitude`); written with pad_dim dims a head."""
    lib = _lib("conv_qkv", proj, q_out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    H, G, dk, dv, D = n_heads, n_kv_heads, k_dim, v_dim, pad_dim
    channels = H * dk + G * (dk + dv)
    if col0 < 0 or col0 + channels > width:
        raise KernelError("the projection is narrower than its q/k/v columns")
    outs = [(q_out, "q_out", H * D)] + ([(k_out, "k_out", G * D), (v_out, "v_out", G * D)] if G else [])
    for t, nm, w in outs:
        _need(t, nm, proj.dtype, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    _f32_vec(q_norm, "q_norm", dk); _f32_vec(k_norm, "k_norm", dk)
    _f32_vec(inv_freq, "inv_freq", rot_dims // 2 if rot_dims else None)
    keep = 0
    if conv_w is not None:
        _need(conv_w, "conv_w", torch.float32, 2)
        if tuple(conv_w.shape) != (taps, channels):
            raise KernelError(f"conv_w must be [{taps}, {channels}]")
        keep = taps - 1
    if keep:
        _need(state, "state", proj.dtype, 3)
        if tuple(state.shape[1:]) != (keep, channels):
            raise KernelError(f"state must be [slots, {keep}, {channels}]")
    for t, nm in ((ctx.token_request, "token_request"), (ctx.positions, "positions"), (ctx.q_start, "q_start"),
                  (ctx.q_len, "q_len"), (ctx.state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    R = ctx.q_len.shape[0]
    update = 0 if (ctx.decode_only or not keep) else 1
    _check(lib.tnx_conv_qkv_prep(_p(proj), c_int(ld), c_int(col0), _p(conv_w), c_int(taps if conv_w is not None else 1),
                                 _p(state if keep else None), _p(ctx.token_request), _p(ctx.positions), _p(ctx.q_start),
                                 _p(ctx.q_len), _p(ctx.state_slots), c_int(R), c_int(update), _p(q_norm), _p(k_norm),
                                 c_float(eps), _p(inv_freq), c_int(rot_dims if inv_freq is not None else 0),
                                 c_int(1 if interleaved else 0), c_float(magnitude), _p(q_out), _p(k_out if G else None),
                                 _p(v_out if G else None), c_int(N), c_int(H), c_int(G), c_int(dk), c_int(dv), c_int(D),
                                 c_int(_is_h16(proj)), _stream()), "conv_qkv_prep")
    add_launches(update)


def moe_route(h, router, token_request, ids, weights, top, softmax_scores=False, renormalize=False, correction=None,
              n_groups=1, keep_groups=1, group_top=2, renorm_eps=0.0, weight_scale=1.0):
    """For every row of h [N, W]: the `top` experts with the largest scores (sigmoid, or softmax, of the 32-bit product
    with router [E, W]) into ids [N, top] (int32; -1 for a padded row) and their scores into weights [N, top].
    correction (32-bit [E]): added to the sigmoid scores for the choice only.  n_groups > 1: the experts form equal groups
    of neighbours, a group's score is the sum of its group_top largest choice scores, and only experts of the keep_groups
    best groups can be chosen.  The weights are divided by (their sum + renorm_eps) with `renormalize`, then multiplied
    by weight_scale."""
    lib = _lib("moe", h, router)
    _need(h, "h", _FLOATS, None, contiguous=False)
    N, W, ld = _rows_2d(h, "h")
    _need(router, "router", _FLOATS, 2)
    E = router.shape[0]
    if router.shape[1] != W:
        raise KernelError("the router's rows must be as long as h's")
    _need(token_request, "token_request", torch.int32, 1)
    _need(ids, "ids", torch.int32, 2); _need(weights, "weights", torch.float32, 2)
    if tuple(ids.shape) != (N, top) or tuple(weights.shape) != (N, top):
        raise KernelError(f"ids and weights must be [{N}, {top}]")
    _f32_vec(correction, "correction", E)
    _check(lib.tnx_moe_route(_p(h), c_int(ld), _p(router), _p(token_request), _p(ids), _p(weights), c_int(N), c_int(W),
                             c_int(E), c_int(top), c_int(1 if softmax_scores else 0), c_int(1 if renormalize else 0),
                             c_int(_is_h16(h)), c_int(_is_h16(router)), _p(correction), c_int(n_groups), c_int(keep_groups),
                             c_int(group_top), c_float(renorm_eps), c_float(weight_scale), _stream()), "moe_route")


EXPERT_FORMS = {"gated_swish": 0, "relu2": 1}


def moe_experts(h, gate_up, down, ids, weights, y, out, gate_max, up_min, up_max, alpha, up_shift, weight_on_input=True,
                accumulate=False, per_pair=None, form="gated_swish"):
    """The chosen experts of every row, an expert's matrices streamed once for every four rows that chose it:
    gate_up [E, 2F, W] (gate rows, then up rows; with form 'relu2', experts without a gate, [E, F, W]: the up rows
    alone), down [E, W, F]; y [N * top, F] scratch in h's type and per_pair [N * top, W] 32-bit scratch (made here when
    not given); out 32-bit [N, W], written or added to."""
    lib = _lib("moe", h, gate_up)
    _need(h, "h", _FLOATS, None, contiguous=False)
    N, W, ld = _rows_2d(h, "h")
    _need(gate_up, "gate_up", _FLOATS, 3); _need(down, "down", gate_up.dtype, 3)
    E, F2, Wg = gate_up.shape
    per = 1 if EXPERT_FORMS[form] else 2
    F = F2 // per
    if Wg != W or F2 % per or tuple(down.shape) != (E, W, F):
        raise KernelError(f"gate_up must be [E, {per}F, {W}] and down [E, {W}, F]")
    top = ids.shape[1]
    _need(ids, "ids", torch.int32, 2); _need(weights, "weights", torch.float32, 2)
    _need(y, "y", h.dtype, 2); _need(out, "out", torch.float32, 2)
    if tuple(ids.shape) != (N, top) or tuple(weights.shape) != (N, top) or tuple(y.shape) != (N * top, F) \
            or tuple(out.shape) != (N, W):
        raise KernelError("ids, weights, y or out do not fit the rows and experts")
    if per_pair is None:
        per_pair = torch.empty((N * top, W), dtype=torch.float32, device=h.device)
    _need(per_pair, "per_pair", torch.float32, 2)
    if tuple(per_pair.shape) != (N * top, W):
        raise KernelError(f"per_pair must be [{N * top}, {W}]")
    _check(lib.tnx_moe_experts(_p(h), c_int(ld), _p(gate_up), _p(down), _p(ids), _p(weights), _p(y), _p(per_pair), _p(out),
                               c_int(N), c_int(W), c_int(F), c_int(top), c_int(E), c_float(gate_max), c_float(up_min),
                               c_float(up_max),
                               c_float(alpha), c_float(up_shift), c_int(1 if weight_on_input else 0),
                               c_int(1 if accumulate else 0), c_int(_is_h16(h)), c_int(_is_h16(gate_up)),
                               c_int(EXPERT_FORMS[form]), _stream()),
           "moe_experts")
    add_launches(2)


def moe_grouped_supported(h, gate_up, down) -> bool:
    """Whether the grouped tensor-core form takes these tensors: a 16-bit engine whose experts are stored in its own
    16-bit type, widths that are multiples of 8 (16-byte row pitches for the TMA descriptors), at most 1024 experts."""
    if h.dtype not in _H16 or gate_up.dtype != h.dtype or down.dtype != h.dtype:
        return False
    E, F2, W = gate_up.shape
    return (W % 8 == 0 and down.shape[2] % 8 == 0 and E <= 1024 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0
            and gate_up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0 and E * max(F2, W) < 2 ** 31)


def gemm_tc_grouped(a, w, out, group_of_tile, tile=128, used_tiles=0):
    """out[m] = a[m] @ w[g]^T for the rows m of every tile of `tile` rows, g = group_of_tile[m // tile] (-1: the tile is
    skipped).  a [M, K] (M a multiple of tile) and w [groups, N, K] in one 16-bit type; out [M, N] in that type or
    32-bit.  tile 128: tiles of 128 tokens x 128 features; 16, 32 or 64: the swapped form (the group's matrix fills the
    128-row operand), K split in clusters while the `used_tiles` tiles expected to have a group leave SMs idle."""
    lib = _lib("gemm_tc", a, w, out)
    _need(a, "a", _H16, 2); _need(w, "w", a.dtype, 3); _need(out, "out", _FLOATS, 2)
    _need(group_of_tile, "group_of_tile", torch.int32, 1)
    M, K = a.shape
    G, N, Kw = w.shape
    if Kw != K or tuple(out.shape) != (M, N) or tile not in (16, 32, 64, 128) or M % tile or group_of_tile.shape[0] < M // tile:
        raise KernelError(f"grouped product shapes do not fit: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    st = _state(a.device)
    if tile < 128:
        _check(lib.tnx_gemm_tc_grouped_few(_p(a), _p(w), _p(out), c_int(M), c_int(N), c_int(K), c_int(G), c_int(tile),
                                           c_int(int(used_tiles)), c_int(K), c_int(K), c_int(N), c_int(_is_h16(out)),
                                           _p(group_of_tile), _p(st["err"]), _stream()), "gemm_tc_grouped")
        return
    _check(lib.tnx_gemm_tc_grouped(_p(a), _p(w), _p(out), c_int(M), c_int(N), c_int(K), c_int(G), c_int(K), c_int(K), c_int(N),
                                   c_int(_is_h16(out)), _p(group_of_tile), _p(st["err"]), _stream()), "gemm_tc_grouped")


def gemm_tc_batched_supported(x, x_head, w, out, out_head) -> bool:
    """What gemm_tc_batched takes: one 16-bit type, head pitches and row pitches that are multiples of 8 elements,
    16-byte aligned bases, and K rounded up to 64 inside a head's own columns of x."""
    if x.dtype not in _H16 or w.dtype != x.dtype or out.dtype != x.dtype or w.dim() != 3 or not w.is_contiguous():
        return False
    H, n_out, k = w.shape
    if k % 8 or x_head % 8 or out_head % 8 or x.stride(0) % 8 or out.stride(0) % 8 or x.stride(1) != 1 or out.stride(1) != 1:
        return False
    if -(-k // 64) * 64 > x_head or out_head < n_out or H * x_head > x.stride(0) or H * out_head > out.stride(0):
        return False
    return x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0


def gemm_tc_batched(x, x_head, w, out, out_head):
    """out[n, h * out_head + c] = sum_i x[n, h * x_head + i] * w[h, c, i] for every head h in ONE launch of the tcgen05
    product (w [heads, n_out, k], 32-bit sums).  The columns of x between k and k rounded up to 64 are read (against
    zeros of w): they must hold finite numbers."""
    lib = _lib("gemm_tc", x, w, out)
    if not gemm_tc_batched_supported(x, x_head, w, out, out_head):
        raise KernelError("gemm_tc_batched: a 16-bit type, pitches that are multiples of 8, 16-byte aligned bases, and k "
                          "rounded up to 64 within a head's columns")
    H, n_out, k = w.shape
    N = x.shape[0]
    if out.shape[0] != N:
        raise KernelError("x and out differ in rows")
    st = _state(x.device)
    _check(lib.tnx_gemm_tc_batched(_p(x), _p(w), _p(out), c_int(N), c_int(n_out), c_int(k), c_int(H), c_int(x.stride(0)),
                                   c_int(x_head), c_int(out.stride(0)), c_int(out_head), c_int(1), _p(st["err"]), _stream()),
           "gemm_tc_batched")


def moe_grouped(ctx, h, gate_up, down, ids, weights, out, gate_max, up_min, up_max, alpha, up_shift, weight_on_input=True,
                accumulate=False, form="gated_swish"):
    """moe_experts for many rows: the (row, expert) pairs sorted by expert into 128-row tiles, the experts' two
    products as grouped tensor-core products, the activation between them and the sum over a row's experts as
    kernels of csrc/moe_grouped.cu.  Buffers come from ctx.scratch; nothing is read on the host."""
    lib = _lib("moe_grouped", h, gate_up)
    if not moe_grouped_supported(h, gate_up, down):
        raise KernelError("the grouped form takes a 16-bit engine, experts stored in its type and widths that are multiples of 8")
    N, W = h.shape
    E, F2, _ = gate_up.shape
    F, top = down.shape[2], ids.shape[1]
    P = N * top
    # the tile: the smallest that holds twice an expert's even share of the pairs (so that most experts take one tile and
    # their matrices are streamed once), 128 rows where the experts get many
    tile = next((t for t in (16, 32, 64) if 2 * P <= t * E), 128)
    tiles = lib.tnx_moe_grouped_max_tiles(c_int(P), c_int(E), c_int(tile))
    used = min(E, P) + P // tile // 2
    rows = tiles * tile
    group_of_tile = ctx.scratch(1, tiles, torch.int32).view(-1)
    row_of_pair = ctx.scratch(1, P, torch.int32).view(-1)
    x = ctx.scratch(rows, W, h.dtype)
    moe_sort_rows(lib, h, ids, weights, E, tiles, tile, group_of_tile, row_of_pair, x, weight_on_input)
    gu = ctx.scratch(rows, F2, h.dtype)
    gemm_tc_grouped(x, gate_up, gu, group_of_tile, tile, used)
    y = ctx.scratch(rows, F, h.dtype)
    moe_activation(lib, gu, y, group_of_tile, tile, gate_max, up_min, up_max, alpha, up_shift, form)
    per_pair = ctx.scratch(rows, W, torch.float32)
    gemm_tc_grouped(y, down, per_pair, group_of_tile, tile, used)
    moe_combine(lib, per_pair, row_of_pair, weights, out, accumulate, weight_on_input)


def moe_sort_rows(lib, h, ids, weights, n_experts, tiles, tile, group_of_tile, row_of_pair, x, weight_on_input):
    """The plan (every pair's row, every tile's expert) and the rows themselves, x[row(pair)] = weight * h[token]."""
    P, top = ids.numel(), ids.shape[1]
    _check(lib.tnx_moe_plan(_p(ids), c_int(P), c_int(n_experts), c_int(tiles), c_int(tile), _p(group_of_tile), _p(row_of_pair),
                            _stream()), "moe_plan")
    _check(lib.tnx_moe_gather(_p(h), c_int(h.stride(0)), _p(weights), _p(row_of_pair), _p(x), c_int(P), c_int(h.shape[1]),
                              c_int(top), c_int(1 if weight_on_input else 0), _stream()), "moe_gather")


def moe_activation(lib, gu, y, group_of_tile, tile, gate_max, up_min, up_max, alpha, up_shift, form="gated_swish"):
    _check(lib.tnx_moe_act(_p(gu), _p(y), _p(group_of_tile), c_int(tile), c_int(gu.shape[0]), c_int(y.shape[1]), c_float(gate_max),
                           c_float(up_min), c_float(up_max), c_float(alpha), c_float(up_shift), c_int(EXPERT_FORMS[form]),
                           _stream()), "moe_act")


def moe_combine(lib, per_pair, row_of_pair, weights, out, accumulate, weight_on_input):
    N, W = out.shape
    _check(lib.tnx_moe_combine(_p(per_pair), _p(row_of_pair), _p(weights), _p(out), c_int(N), c_int(W), c_int(weights.shape[1]),
                               c_int(1 if accumulate else 0), c_int(1 if weight_on_input else 0), _stream()), "moe_combine")


def rotary_qkv_prep(proj, q_off, k_off, v_off, token_request, positions, q_weight, k_weight, eps, head_scale,
                    inv_freq_qk, rot_dims, inv_freq_v, q_out, k_out, v_out, n_heads, n_kv_heads, k_dim, v_dim, pad_dim):
    """From one product's output `proj` [N, *] (queries at column q_off, keys at k_off, values at v_off): the
    queries and keys normalised over the whole projection (where a weight is given), rotated by position
    on their first rot_dims dims, the queries multiplied by their head's number; the values rotated over
    all their dims (where inv_freq_v is given); each written with pad_dim dims a head, the rest zero."""
    lib = _lib("rotary_qkv", proj, q_out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    H, G, dk, dv, D = n_heads, n_kv_heads, k_dim, v_dim, pad_dim
    if max(q_off + H * dk, k_off + G * dk, v_off + G * dv) > width:
        raise KernelError("the projection is narrower than its q/k/v columns")
    for t, nm, w in ((q_out, "q_out", H * D), (k_out, "k_out", G * D), (v_out, "v_out", G * D)):
        _need(t, nm, proj.dtype, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    _f32_vec(q_weight, "q_weight", H * dk); _f32_vec(k_weight, "k_weight", G * dk); _f32_vec(head_scale, "head_scale", H)
    _f32_vec(inv_freq_qk, "inv_freq_qk", rot_dims // 2 if rot_dims else None); _f32_vec(inv_freq_v, "inv_freq_v", dv // 2)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_rotary_qkv_prep(_p(proj), c_int(ld), c_int(q_off), c_int(k_off), c_int(v_off), _p(token_request),
                                   _p(positions), _p(q_weight), _p(k_weight), c_float(eps), _p(head_scale),
                                   _p(inv_freq_qk), c_int(rot_dims), _p(inv_freq_v), _p(q_out), _p(k_out), _p(v_out),
                                   c_int(N), c_int(H), c_int(G), c_int(dk), c_int(dv), c_int(D), c_int(_is_h16(proj)),
                                   _stream()), "rotary_qkv_prep")


def rotary_unrotate(att, token_request, positions, inv_freq_v, out_scale, out, n_heads, v_dim, pad_dim):
    """att [N, n_heads * pad_dim]: each head's first v_dim dims turned back by the token's position (pair m with
    m + v_dim/2, by -p * inv_freq_v[m]; no turn without inv_freq_v), times out_scale, written v_dim a head into
    `out` [N, n_heads * v_dim] (a column slice of a wider buffer is allowed)."""
    lib = _lib("rotary_qkv", att, out)
    _need(att, "att", _FLOATS, 2)
    N = att.shape[0]
    if att.shape[1] != n_heads * pad_dim:
        raise KernelError("att must hold pad_dim dims a head")
    _need(out, "out", att.dtype, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (No, wo) != (N, n_heads * v_dim):
        raise KernelError(f"out must be [{N}, {n_heads * v_dim}]")
    _f32_vec(inv_freq_v, "inv_freq_v", v_dim // 2)
    _check(lib.tnx_rotary_unrotate(_p(att), _p(token_request), _p(positions), _p(inv_freq_v), c_float(out_scale),
                                   _p(out), c_int(out_ld), c_int(N), c_int(n_heads), c_int(v_dim), c_int(pad_dim),
                                   c_int(_is_h16(att)), _stream()), "rotary_unrotate")


def retention_prep(proj, q_off, k_off, token_request, positions, inv_freq, rot_dims, k_scale, q_out, k_out, n_heads, k_dim):
    """32-bit queries and keys [N, n_heads * k_dim] for the retention scan: rotated by position on their first
    rot_dims dims, the keys then multiplied by k_scale."""
    lib = _lib("retention", proj)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    if max(q_off, k_off) + n_heads * k_dim > width:
        raise KernelError("the projection is narrower than its q/k columns")
    for t, nm in ((q_out, "q_out"), (k_out, "k_out")):
        _need(t, nm, torch.float32, 2)
        if tuple(t.shape) != (N, n_heads * k_dim):
            raise KernelError(f"{nm} must be [{N}, {n_heads * k_dim}]")
    _f32_vec(inv_freq, "inv_freq", rot_dims // 2 if rot_dims else None)
    _check(lib.tnx_retention_prep(_p(proj), c_int(ld), c_int(q_off), c_int(k_off), _p(token_request), _p(positions),
                                  _p(inv_freq), c_int(rot_dims), c_float(k_scale), _p(q_out), _p(k_out), c_int(N),
                                  c_int(n_heads), c_int(k_dim), c_int(_is_h16(proj)), _stream()), "retention_prep")


def retention_scan(q, k, v, decay, state, q_start, q_len, state_slots, out, n_heads, k_dim, v_dim, most_tokens=None,
                   decay_tok=None, kscale_tok=None, qk_heads=None):
    """S <- decay S + k v^T, o = S^T q, token by token for every request of the step (q_start, q_len: its rows;
    q_len 0 or slot < 0: skipped).  q, k: 32-bit [N, n_heads * k_dim]; v: [N, n_heads * v_dim] view in the
    activation type or 32-bit; state: 32-bit [slots, n_heads, v_dim, k_dim]; out: 32-bit [N, n_heads * v_dim].
    most_tokens: an upper bound of any request's rows (default: N); a step of single tokens says 1 and gets
    small stages.  decay_tok, kscale_tok (32-bit [N, n_heads]): S <- decay_tok S + kscale_tok k v^T with numbers of the
    token (absent: decay[h], 1); qk_heads: q and k are [N, qk_heads * k_dim] and head h reads those of
    h // (n_heads // qk_heads)."""
    lib = _lib("retention", v)
    N = q.shape[0]
    qk_heads = n_heads if qk_heads is None else int(qk_heads)
    if qk_heads <= 0 or n_heads % qk_heads:
        raise KernelError(f"{n_heads} heads cannot share {qk_heads} heads of queries and keys")
    for t, nm in ((decay_tok, "decay_tok"), (kscale_tok, "kscale_tok")):
        if t is not None:
            _need(t, nm, torch.float32, 2)
            if tuple(t.shape) != (N, n_heads):
                raise KernelError(f"{nm} must be [{N}, {n_heads}]")
    if decay is None and decay_tok is None:
        raise KernelError("a decay per head or per token is needed")
    for t, nm in ((q, "q"), (k, "k")):
        _need(t, nm, torch.float32, 2)
        if tuple(t.shape) != (N, qk_heads * k_dim):
            raise KernelError(f"{nm} must be [{N}, {qk_heads * k_dim}]")
    _need(v, "v", _FLOATS, None, contiguous=False)
    Nv, wv, v_ld = _rows_2d(v, "v")
    if (Nv, wv) != (N, n_heads * v_dim):
        raise KernelError(f"v must be [{N}, {n_heads * v_dim}]")
    _need(state, "state", torch.float32, 4)
    if tuple(state.shape[1:]) != (n_heads, v_dim, k_dim):
        raise KernelError(f"state must be [slots, {n_heads}, {v_dim}, {k_dim}]")
    _need(out, "out", torch.float32, 2)
    if tuple(out.shape) != (N, n_heads * v_dim):
        raise KernelError(f"out must be [{N}, {n_heads * v_dim}]")
    _f32_vec(decay, "decay", n_heads)
    for t, nm in ((q_start, "q_start"), (q_len, "q_len"), (state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    R = q_len.shape[0]
    if q_start.shape[0] < R or state_slots.shape[0] < R:
        raise KernelError("q_start and state_slots must cover every request of q_len")
    _check(lib.tnx_retention_scan(_p(q), _p(k), _p(v), c_int(v_ld), _p(decay), _p(state), _p(q_start), _p(q_len),
                                  _p(state_slots), _p(out), c_int(R), c_int(n_heads), c_int(k_dim), c_int(v_dim),
                                  c_int(max(1, int(most_tokens if most_tokens is not None else N))), c_int(_is_h16(v)),
                                  _p(decay_tok), _p(kscale_tok), c_int(qk_heads), _stream()), "retention_scan")


def retention_decode(proj, q_off, k_off, v_off, g_off, positions, inv_freq, rot_dims, k_scale, decay, state, q_start, q_len,
                     state_slots, eps, out_scale, out, n_heads, k_dim, v_dim) -> bool:
    """A step in which every request has ONE row: retention_prep, retention_scan and headwise_gated_rms_norm in one
    kernel (the 32-bit queries, keys and outputs never pass through memory).  Returns False, having launched nothing,
    for sizes the kernel does not take (k_dim or v_dim no multiple of four, very wide heads): the caller then runs the
    three kernels.  g_off None: no gate."""
    lib = _lib("retention", proj, out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    offs = [q_off + n_heads * k_dim, k_off + n_heads * k_dim, v_off + n_heads * v_dim] + \
           ([g_off + n_heads * v_dim] if g_off is not None else [])
    if max(offs) > width:
        raise KernelError("the projection is narrower than its q/k/v/gate columns")
    _need(state, "state", torch.float32, 4)
    if tuple(state.shape[1:]) != (n_heads, v_dim, k_dim):
        raise KernelError(f"state must be [slots, {n_heads}, {v_dim}, {k_dim}]")
    _need(out, "out", proj.dtype, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (No, wo) != (N, n_heads * v_dim):
        raise KernelError(f"out must be [{N}, {n_heads * v_dim}]")
    _f32_vec(decay, "decay", n_heads)
    _f32_vec(inv_freq, "inv_freq", rot_dims // 2 if rot_dims else None)
    for t, nm in ((positions, "positions"), (q_start, "q_start"), (q_len, "q_len"), (state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    code = lib.tnx_retention_decode(_p(proj), c_int(ld), c_int(q_off), c_int(k_off), c_int(v_off),
                                    c_int(-1 if g_off is None else g_off), _p(positions), _p(inv_freq), c_int(rot_dims),
                                    c_float(k_scale), _p(decay), _p(state), _p(q_start), _p(q_len), _p(state_slots),
                                    c_float(eps), c_float(out_scale), _p(out), c_int(out_ld), c_int(q_len.shape[0]),
                                    c_int(n_heads), c_int(k_dim), c_int(v_dim), c_int(_is_h16(proj)), _stream())
    if code == -2:
        return False
    _check(code, "retention_decode")
    return True


def retention_scan_force(lanes=0, stage_tokens=0, dtype=None) -> None:
    """A test and measurement hook: the lanes a column's rows are spread over (0: the kernel's own choice; 16 for key
    sizes of 65 to 128) and the most tokens of a stage (0: the kernel's own choice, which follows the number of blocks).
    `dtype`: which flavour of the library (the 16-bit type of the values it will be given; None: bfloat16's)."""
    lib = _build.load("retention", dtype if dtype in _H16 else None)
    if lib.tnx_retention_scan_force(c_int(int(lanes)), c_int(int(stage_tokens))) != 0:
        raise KernelError(f"retention_scan_force: {lanes} lanes (0 or 16) and stages of {stage_tokens} tokens (0 to 32) are not a choice")


def headwise_gated_rms_norm(o, gate, token_request, weight, eps, out_scale, out, n_heads, v_dim, gate_activation="silu"):
    """out = o / rms(o over each head's v_dim dims) (* weight) * act(gate) * out_scale; o 32-bit [N, n_heads * v_dim],
    gate (optional) and out views in the activation type; act: silu unless named otherwise."""
    lib = _lib("retention", gate, out)
    _need(o, "o", torch.float32, 2)
    N = o.shape[0]
    if o.shape[1] != n_heads * v_dim:
        raise KernelError(f"o must be [{N}, {n_heads * v_dim}]")
    gate_ld = 0
    if gate is not None:
        _need(gate, "gate", out.dtype, None, contiguous=False)
        Ng, wg, gate_ld = _rows_2d(gate, "gate")
        if (Ng, wg) != (N, n_heads * v_dim):
            raise KernelError(f"gate must be [{N}, {n_heads * v_dim}]")
    _need(out, "out", _FLOATS, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (No, wo) != (N, n_heads * v_dim):
        raise KernelError(f"out must be [{N}, {n_heads * v_dim}]")
    _f32_vec(weight, "weight", v_dim)
    _check(lib.tnx_headwise_gated_rms_norm(_p(o), _p(gate), c_int(gate_ld), _p(token_request), _p(weight), c_float(eps),
                                           c_float(out_scale), _p(out), c_int(out_ld), c_int(N), c_int(n_heads),
                                           c_int(v_dim), c_int(activation_code(gate_activation)), c_int(_is_h16(out)),
                                           _stream()), "headwise_gated_rms_norm")


def ssd_prep(proj, col0, conv_w, conv_b, taps, state, ctx, a_log, dt_bias, activation, x_out, b_out, c_out, dt_out,
             decay_out, n_heads, v_dim, groups, state_dim):
    """From the input projection's output `proj` [N, *] (from column col0 on: z | x | B | C | dt): x, B and C through
    their short causal convolution (conv_w [taps, channels], conv_b [channels] or None, both 32-bit; state
    [slots, taps - 1, channels] in proj's type) and the activation, as 32-bit x [N, heads * v_dim], B and C
    [N, groups * state_dim]; dt = softplus(dt + dt_bias) and decay = exp(-exp(a_log) dt), 32-bit [N, heads]."""
    lib = _lib("ssd", proj)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    H, P, G, Ns = n_heads, v_dim, groups, state_dim
    inner, C = H * P, H * P + 2 * G * Ns
    if col0 < 0 or col0 + inner + C + H > width:
        raise KernelError("the projection is narrower than its columns")
    _need(conv_w, "conv_w", torch.float32, 2)
    if tuple(conv_w.shape) != (taps, C):
        raise KernelError(f"conv_w must be [{taps}, {C}]")
    _f32_vec(conv_b, "conv_b", C); _f32_vec(a_log, "a_log", H); _f32_vec(dt_bias, "dt_bias", H)
    if taps > 1:
        _need(state, "state", proj.dtype, 3)
        if tuple(state.shape[1:]) != (taps - 1, C):
            raise KernelError(f"state must be [slots, {taps - 1}, {C}]")
    for t, nm, w in ((x_out, "x_out", inner), (b_out, "b_out", G * Ns), (c_out, "c_out", G * Ns), (dt_out, "dt_out", H),
                     (decay_out, "decay_out", H)):
        _need(t, nm, torch.float32, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    for t, nm in ((ctx.token_request, "token_request"), (ctx.positions, "positions"), (ctx.q_start, "q_start"),
                  (ctx.q_len, "q_len"), (ctx.state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    _check(lib.tnx_ssd_prep(_p(proj), c_int(ld), c_int(col0), _p(conv_w), _p(conv_b), c_int(taps),
                            _p(state if taps > 1 else None), _p(ctx.token_request), _p(ctx.positions), _p(ctx.q_start),
                            _p(ctx.q_len), _p(ctx.state_slots), _p(a_log), _p(dt_bias), c_int(activation_code(activation)),
                            _p(x_out), _p(b_out), _p(c_out), _p(dt_out), _p(decay_out), c_int(N), c_int(H), c_int(P),
                            c_int(G), c_int(Ns), c_int(_is_h16(proj)), _stream()), "ssd_prep")
    if taps > 1 and not ctx.decode_only:
        conv_state_update(proj, col0 + inner, state, ctx)


def ssd_gate_norm(y, x, skip, z, token_request, weight, eps, activation, out, v_dim, parts):
    """out = rms_in_parts((y + skip[head] * x) * act(z)) * weight: y and x 32-bit [N, inner], z and out views in the
    activation type, the root mean square taken over each of `parts` equal parts of the inner width."""
    lib = _lib("ssd", z, out)
    _need(y, "y", torch.float32, 2)
    N, inner = y.shape
    if skip is not None:
        _need(x, "x", torch.float32, 2)
        if tuple(x.shape) != (N, inner) or inner % v_dim:
            raise KernelError(f"x must be [{N}, {inner}]")
        _f32_vec(skip, "skip", inner // v_dim)
    _need(z, "z", out.dtype, None, contiguous=False)
    Nz, wz, z_ld = _rows_2d(z, "z")
    _need(out, "out", _FLOATS, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (Nz, wz) != (N, inner) or (No, wo) != (N, inner):
        raise KernelError(f"z and out must be [{N}, {inner}]")
    _f32_vec(weight, "weight", inner)
    _check(lib.tnx_ssd_gate_norm(_p(y), _p(x), _p(skip), _p(z), c_int(z_ld), _p(token_request), _p(weight), c_float(eps),
                                 c_int(activation_code(activation)), _p(out), c_int(out_ld), c_int(N), c_int(inner),
                                 c_int(v_dim), c_int(parts), c_int(_is_h16(out)), _stream()), "ssd_gate_norm")


def diff_qkv_prep(proj, col0, token_request, positions, q_norm, k_norm, eps, temp_coef, temp_every, q_out, k_out, v_out,
                  n_heads, n_kv_heads, k_dim, v_dim, pad_dim):
    """Queries, keys and values of differential attention from one product's output `proj` [N, *] (from column col0 on:
    queries [heads][2][k_dim], then, unless n_kv_heads is 0, keys [kv_heads][2][k_dim] and values [kv_heads][v_dim]):
    per head and map an RMS norm with one weight vector (q_norm, k_norm [k_dim]; None: no weight), queries times
    1 + temp_coef ln(floor((p + 1) / temp_every) + 1) (temp_every 0: not), written for ONE paged attention call with
    2 heads query heads of pad_dim dims: q_out [N, 2 heads * pad_dim] (map m of a head in columns m k_dim ..), k_out
    [N, kv_heads * pad_dim] (both maps side by side), v_out the same shape."""
    lib = _lib("diff_attention", proj, q_out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    H, G, dk, dv, D = n_heads, n_kv_heads, k_dim, v_dim, pad_dim
    if col0 < 0 or col0 + 2 * H * dk + G * (2 * dk + dv) > width:
        raise KernelError("the projection is narrower than its q/k/v columns")
    outs = [(q_out, "q_out", 2 * H * D)] + ([(k_out, "k_out", G * D), (v_out, "v_out", G * D)] if G else [])
    for t, nm, w in outs:
        _need(t, nm, proj.dtype, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    _f32_vec(q_norm, "q_norm", dk); _f32_vec(k_norm, "k_norm", dk)
    _need(token_request, "token_request", torch.int32, 1); _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_diff_qkv_prep(_p(proj), c_int(ld), c_int(col0), _p(token_request), _p(positions), _p(q_norm), _p(k_norm),
                                 c_float(eps), c_float(temp_coef), c_int(temp_every), _p(q_out), _p(k_out if G else None),
                                 _p(v_out if G else None), c_int(N), c_int(H), c_int(G), c_int(dk), c_int(dv), c_int(D),
                                 c_int(_is_h16(proj)), _stream()), "diff_qkv_prep")


def diff_combine(att, gate, token_request, lam, eps, out_mult, out_scale, out, n_heads, v_dim, pad_dim):
    """From the attention's output att [N, 2 heads * pad_dim] (query head 2 h + map): o = a1 - lam a2 over the first v_dim
    dims, divided by its root mean square, times out_mult, times sigmoid(gate[n, h]) (gate [N, heads] view or None),
    times out_scale, into out [N, heads * v_dim] (a view with contiguous rows)."""
    lib = _lib("diff_attention", att, out)
    _need(att, "att", _FLOATS, 2)
    N = att.shape[0]
    if att.shape[1] != 2 * n_heads * pad_dim:
        raise KernelError(f"att must be [{N}, {2 * n_heads * pad_dim}]")
    gate_ld = 0
    if gate is not None:
        _need(gate, "gate", att.dtype, None, contiguous=False)
        Ng, wg, gate_ld = _rows_2d(gate, "gate")
        if (Ng, wg) != (N, n_heads):
            raise KernelError(f"gate must be [{N}, {n_heads}]")
    _need(out, "out", att.dtype, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (No, wo) != (N, n_heads * v_dim):
        raise KernelError(f"out must be [{N}, {n_heads * v_dim}]")
    _check(lib.tnx_diff_combine(_p(att), _p(gate), c_int(gate_ld), _p(token_request), c_float(lam), c_float(eps),
                                c_float(out_mult), c_float(out_scale), _p(out), c_int(out_ld), c_int(N), c_int(n_heads),
                                c_int(v_dim), c_int(pad_dim), c_int(_is_h16(att)), _stream()), "diff_combine")


def mingru_scan(proj, z_off, x_off, g_off, state, q_start, q_len, state_slots, out, width, out_scale=1.0,
                most_tokens=None):
    """The minGRU recurrence over every request's rows of the step, from the raw projections in `proj` [N, *]
    (update gate at column z_off, candidate at x_off, output gate at g_off or None); state 32-bit [slots, width];
    out [N, width] in proj's type: the new state times silu(output gate) times out_scale.  most_tokens: an upper
    bound of any request's rows (default: N); it decides over how many warps a request's tokens are spread."""
    lib = _lib("mingru", proj, out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, wide, ld = _rows_2d(proj, "proj")
    offs = [z_off, x_off] + ([g_off] if g_off is not None else [])
    if max(offs) + width > wide or min(offs) < 0:
        raise KernelError("the projection is narrower than its gate columns")
    _need(state, "state", torch.float32, 2)
    if state.shape[1] != width:
        raise KernelError(f"state must be [slots, {width}]")
    _need(out, "out", proj.dtype, None, contiguous=False)
    No, wo, out_ld = _rows_2d(out, "out")
    if (No, wo) != (N, width):
        raise KernelError(f"out must be [{N}, {width}]")
    for t, nm in ((q_start, "q_start"), (q_len, "q_len"), (state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    R = q_len.shape[0]
    _check(lib.tnx_mingru_scan(_p(proj), c_int(ld), c_int(z_off), c_int(x_off), c_int(-1 if g_off is None else g_off),
                               _p(state), _p(q_start), _p(q_len), _p(state_slots), _p(out), c_int(out_ld), c_float(out_scale),
                               c_int(R), c_int(width), c_int(max(1, int(most_tokens if most_tokens is not None else N))),
                               c_int(_is_h16(proj)), _stream()), "mingru_scan")


def gated_activation(gate_up, out, activation):
    """out = act(gate_up[:, :F]) * gate_up[:, F:], F = out's width."""
    lib = _lib("gated_act", gate_up, out)
    _need(gate_up, "gate_up", _FLOATS, None, contiguous=False)
    N, wide, ld = _rows_2d(gate_up, "gate_up")
    _need(out, "out", gate_up.dtype, None, contiguous=False)
    No, F, out_ld = _rows_2d(out, "out")
    if No != N or wide != 2 * F:
        raise KernelError(f"gate_up must be [{No}, {2 * F}]")
    _check(lib.tnx_gated_activation(_p(gate_up), c_int(ld), _p(out), c_int(out_ld), c_int(N), c_int(F),
                                    c_int(activation_code(activation)), c_int(_is_h16(out)), _stream()), "gated_activation")


# ---------------------------------------------------------------------------------------------
# Attention through low-rank latents; the recurrence with an error-correcting write.
def latent_prep(proj, col0, token_request, positions, q_norm, kv_norm, eps, inv_freq, interleaved, cq_out, k_out, v_out,
                q_rank, kv_rank, rot_dim):
    """From the down projections' output `proj` [N, *] (from column col0 on: q_rank, kv_rank, rot_dim columns): the
    queries' latent normalised (times q_norm) into cq_out [N, q_rank]; the keys'/values' latent normalised (times
    kv_norm) into the first kv_rank dims of k_out and v_out [N, D]; the rotated key part turned by position behind it
    in k_out; the rest of both rows zero."""
    lib = _lib("latent_attention", proj, cq_out)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    if col0 < 0 or col0 + q_rank + kv_rank + rot_dim > width:
        raise KernelError("the projection is narrower than its latent columns")
    _need(cq_out, "cq_out", proj.dtype, 2)
    _need(k_out, "k_out", proj.dtype, 2)
    _need(v_out, "v_out", proj.dtype, 2)
    D = k_out.shape[1]
    if tuple(cq_out.shape) != (N, q_rank) or tuple(k_out.shape) != (N, D) or tuple(v_out.shape) != (N, D):
        raise KernelError("cq_out must be [N, q_rank], k_out and v_out [N, D]")
    _f32_vec(q_norm, "q_norm", q_rank); _f32_vec(kv_norm, "kv_norm", kv_rank)
    _f32_vec(inv_freq, "inv_freq", rot_dim // 2 if rot_dim else None)
    _need(token_request, "token_request", torch.int32, 1)
    _need(positions, "positions", torch.int32, 1)
    _check(lib.tnx_latent_prep(_p(proj), c_int(ld), c_int(col0), _p(token_request), _p(positions), _p(q_norm), _p(kv_norm),
                               c_float(eps), _p(inv_freq), c_int(1 if interleaved else 0), _p(cq_out), _p(k_out), _p(v_out),
                               c_int(N), c_int(q_rank), c_int(kv_rank), c_int(rot_dim if inv_freq is not None else 0),
                               c_int(D), c_int(_is_h16(proj)), _stream()), "latent_prep")


def headwise_product(x, x_head, w, out, out_head, token_request, n_heads, k, n_out, positions=None, inv_freq=None,
                     rot_dims=0, interleaved=False, pad_to=0, do_product=True):
    """out[n, h * out_head + c] = sum_i x[n, h * x_head + i] * w[h, i, c] (i < k, c < n_out), 32-bit sums; x, w and out in
    one type; w [n_heads, k, n_out].  rot_dims > 0: the head's next rot_dims inputs are turned by the token's position
    into the columns behind n_out, and the head's columns up to pad_to are zeroed.  do_product False: only that."""
    lib = _lib("latent_attention", x, out)
    _need(x, "x", _FLOATS, None, contiguous=False)
    _need(out, "out", x.dtype, None, contiguous=False)
    N, wx, x_ld = _rows_2d(x, "x")
    No, wo, out_ld = _rows_2d(out, "out")
    if No != N or wx < (n_heads - 1) * x_head + k + rot_dims or wo < (n_heads - 1) * out_head + max(n_out, pad_to):
        raise KernelError("x or out is narrower than its heads")
    if do_product:
        _need(w, "w", x.dtype, 3)
        if tuple(w.shape) != (n_heads, k, n_out):
            raise KernelError(f"w must be [{n_heads}, {k}, {n_out}]")
    _need(token_request, "token_request", torch.int32, 1)
    if rot_dims:
        _need(positions, "positions", torch.int32, 1)
        _f32_vec(inv_freq, "inv_freq", rot_dims // 2)
    _check(lib.tnx_headwise_product(_p(x), c_int(x_ld), c_int(x_head), _p(w if do_product else None), _p(out), c_int(out_ld),
                                    c_int(out_head), _p(token_request), _p(positions), _p(inv_freq), c_int(rot_dims),
                                    c_int(1 if interleaved else 0), c_int(pad_to), c_int(1 if do_product else 0), c_int(N),
                                    c_int(n_heads), c_int(k), c_int(n_out), c_int(_is_h16(x)), _stream()), "headwise_product")


def conv_state_update(proj, col0, state, ctx):
    """The convolution state [slots, keep, channels] of every request with more than one row becomes its last `keep`
    projected values (columns col0 .. col0 + channels of proj); requests with one row are left alone."""
    lib = _lib("conv_qkv", proj, state)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    _need(state, "state", proj.dtype, 3)
    keep, channels = state.shape[1], state.shape[2]
    if col0 < 0 or col0 + channels > width:
        raise KernelError("the projection is narrower than the state's channels")
    _check(lib.tnx_conv_state_update(_p(proj), c_int(ld), c_int(col0), _p(state), c_int(keep), c_int(channels),
                                     _p(ctx.q_start), _p(ctx.q_len), _p(ctx.state_slots), c_int(ctx.q_len.shape[0]),
                                     c_int(_is_h16(proj)), _stream()), "conv_state_update")


def delta_prep(proj, col0, b_off, a, conv_w, taps, state, ctx, a_log, dt_bias, unit_eps, q_scale, activation, q_out, k_out,
               v_out, beta_out, g_out, n_heads, n_kv_heads, k_dim, v_dim):
    """From the projections' output `proj` [N, *] (queries, keys, values side by side from column col0 on; the write
    strengths' logits at b_off) and the decays' logits `a` [N, n_heads * k_dim] (32-bit): convolution (conv_w
    [taps, channels] 32-bit, state [slots, taps - 1, channels] in proj's type) and activation, unit-norm q (times q_scale)
    and k, beta = sigmoid, g = exp(-exp(a_log) softplus(a + dt_bias)); all outputs 32-bit."""
    lib = _lib("delta_rule", proj)
    _need(proj, "proj", _FLOATS, None, contiguous=False)
    N, width, ld = _rows_2d(proj, "proj")
    H, G, dk, dv = n_heads, n_kv_heads, k_dim, v_dim
    C = 2 * G * dk + H * dv
    if col0 < 0 or col0 + C > width or b_off < 0 or b_off + H > width:
        raise KernelError("the projection is narrower than its columns")
    _need(a, "a", torch.float32, None, contiguous=False)
    if _rows_2d(a, "a")[:2] != (N, H * dk):
        raise KernelError(f"a must be [{N}, {H * dk}]")
    _need(conv_w, "conv_w", torch.float32, 2)
    if tuple(conv_w.shape) != (taps, C):
        raise KernelError(f"conv_w must be [{taps}, {C}]")
    if taps > 1:
        _need(state, "state", proj.dtype, 3)
        if tuple(state.shape[1:]) != (taps - 1, C):
            raise KernelError(f"state must be [slots, {taps - 1}, {C}]")
    _f32_vec(a_log, "a_log", H); _f32_vec(dt_bias, "dt_bias", H * dk)
    for t, nm, w in ((q_out, "q_out", G * dk), (k_out, "k_out", G * dk), (v_out, "v_out", H * dv), (beta_out, "beta_out", H),
                     (g_out, "g_out", H * dk)):
        _need(t, nm, torch.float32, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    for t, nm in ((ctx.token_request, "token_request"), (ctx.positions, "positions"), (ctx.q_start, "q_start"),
                  (ctx.q_len, "q_len"), (ctx.state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    _check(lib.tnx_delta_prep(_p(proj), c_int(ld), c_int(col0), c_int(b_off), _p(a), c_int(a.stride(0)), _p(conv_w),
                              c_int(taps), _p(state if taps > 1 else None), _p(ctx.token_request), _p(ctx.positions),
                              _p(ctx.q_start), _p(ctx.q_len), _p(ctx.state_slots), _p(a_log), _p(dt_bias), c_float(unit_eps),
                              c_float(q_scale), c_int(activation_code(activation)), _p(q_out), _p(k_out), _p(v_out),
                              _p(beta_out), _p(g_out), c_int(N), c_int(H), c_int(G), c_int(dk), c_int(dv),
                              c_int(_is_h16(proj)), _stream()), "delta_prep")
    if taps > 1 and not ctx.decode_only:
        conv_state_update(proj, col0, state, ctx)


def delta_scan(q, k, v, beta, g, state, q_start, q_len, state_slots, out, n_heads, n_kv_heads, k_dim, v_dim):
    """Per request and head, over the request's rows of this step in order: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    out = S^T q.  All 32-bit; state [slots, n_heads, v_dim, k_dim]; q, k [N, n_kv_heads * k_dim]."""
    lib = _build.load("delta_rule")
    N = q.shape[0]
    for t, nm, w in ((q, "q", n_kv_heads * k_dim), (k, "k", n_kv_heads * k_dim), (v, "v", n_heads * v_dim),
                     (beta, "beta", n_heads), (g, "g", n_heads * k_dim), (out, "out", n_heads * v_dim)):
        _need(t, nm, torch.float32, 2)
        if tuple(t.shape) != (N, w):
            raise KernelError(f"{nm} must be [{N}, {w}]")
    _need(state, "state", torch.float32, 4)
    if tuple(state.shape[1:]) != (n_heads, v_dim, k_dim):
        raise KernelError(f"state must be [slots, {n_heads}, {v_dim}, {k_dim}]")
    for t, nm in ((q_start, "q_start"), (q_len, "q_len"), (state_slots, "state_slots")):
        _need(t, nm, torch.int32, 1)
    _check(lib.tnx_delta_scan(_p(q), _p(k), _p(v), _p(beta), _p(g), _p(state), _p(q_start), _p(q_len), _p(state_slots),
                              _p(out), c_int(q_len.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(k_dim), c_int(v_dim),
                              _stream()), "delta_scan")
