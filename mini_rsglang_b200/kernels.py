"""Python face of the engine's CUDA kernels.

Every function checks its tensors (device, dtype, contiguity, sizes) on the host and then
calls one `extern "C"` launcher of the in-tree kernel library with raw pointers and the
current CUDA stream.  There is no other implementation behind these names: without a GPU,
or without the compiled library, they raise `BackendError`."""
from __future__ import annotations

import ctypes
import math
import os

import torch

from .csrc.build import kernel_library, specialised_kernel_library
from .errors import BackendError, InvalidRequest

_c_int, _c_vp, _c_float = ctypes.c_int, ctypes.c_void_p, ctypes.c_float

_SIGNATURES = {
    "mrs_embed": [_c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_patch_tokens": [_c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_add_rmsnorm": [_c_int, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_rmsnorm": [_c_int, _c_vp, _c_vp, _c_float, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_qk_norm_rope_store": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_vp,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_rotation_table": [_c_vp, _c_vp, _c_int, _c_int, _c_vp, _c_vp],
    "mrs_silu_mul": [_c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_attention_simt": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_float, _c_int, _c_vp],
    "mrs_gemm_f32": [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_argmax": [_c_vp, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_sample": [_c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp],
}

_lib = None
_error_readers: list[tuple] = []
launch_count = 0   # launches of the engine's own kernels since import (read by the benchmark)


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = kernel_library()
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
        lib.mrs_error_string.argtypes = [_c_int]
        lib.mrs_error_string.restype = ctypes.c_char_p
        _lib = lib
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)      # the current stream without building an object for it


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise BackendError(f"{what}: {library().mrs_error_string(code).decode()} (code {code})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, what: str, shape: tuple | None = None) -> None:
    if t.is_cuda and (dtype is None or t.dtype == dtype) and t.is_contiguous() and (shape is None or t.shape == shape):
        return                 # the usual case, in one line: this runs a hundred times a step
    if not t.is_cuda:
        raise BackendError(f"{what}: tensor is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise InvalidRequest(f"{what}: dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise InvalidRequest(f"{what}: tensor is not contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise InvalidRequest(f"{what}: shape {tuple(t.shape)}, expected {tuple(shape)}")


_sm_counts: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (asked once): what launch plans fill."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def check_rotation(head_dim: int, rotary_dim: int, pairing: str, magnitude: float) -> None:
    """Refuses a rotation that the kernels do not compute.  They rotate every element of a head, element j
    with element j + head_dim / 2, by angles position * frequency, cosines and sines unscaled."""
    if pairing != "split_half":
        raise InvalidRequest(f"rotation pairing {pairing!r} is not built; the kernels pair element j with j + head_dim / 2 (\"split_half\")")
    if int(rotary_dim) != int(head_dim):
        raise InvalidRequest(f"a rotation of {rotary_dim} of a head's {head_dim} elements is not built; the kernels rotate whole heads")
    if float(magnitude) != 1.0:
        raise InvalidRequest(f"a rotation whose cosines and sines are scaled by {magnitude} is not built")


def _is_bf16(dtype: torch.dtype) -> int:
    if dtype is torch.bfloat16:
        return 1
    if dtype is torch.float32:
        return 0
    raise InvalidRequest(f"activations must be bfloat16 or float32, got {dtype}")


def embed(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t, :] = float32(table[ids[t], :])."""
    tokens, width = residual.shape
    _need(table, None, "embed table")
    _need(ids, torch.int32, "embed ids", (tokens,))
    _need(residual, torch.float32, "embed output")
    if table.shape[1] != width:
        raise InvalidRequest("embed: width mismatch")
    _check(library().mrs_embed(_is_bf16(table.dtype), table.data_ptr(), ids.data_ptr(), residual.data_ptr(),
                               tokens, width, _stream()), "embed")


def patch_tokens(ids: torch.Tensor, rows: torch.Tensor, index: torch.Tensor, sampled: torch.Tensor, vocab: int) -> None:
    """ids[rows[i]] = sampled[index[i]]: the tokens that the step before sampled go into this step's ids on the
    device, before the host has read them."""
    global launch_count
    n = rows.shape[0]
    _need(ids, torch.int32, "token ids")
    _need(rows, torch.int32, "rows", (n,))
    _need(index, torch.int32, "index", (n,))
    _need(sampled, torch.int32, "sampled tokens")
    launch_count += 1
    _check(library().mrs_patch_tokens(ids.data_ptr(), rows.data_ptr(), index.data_ptr(), sampled.data_ptr(), n, int(vocab),
                                      _stream()), "patch_tokens")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, write_back: bool = True) -> None:
    """v = residual (+ delta); residual = v when write_back; out = norm(v) * weight.
    With `rows`, out[i] comes from source row rows[i]."""
    n_rows, width = out.shape
    _need(residual, torch.float32, "add_rmsnorm residual")
    _need(weight, torch.float32, "add_rmsnorm weight", (width,))
    _need(out, None, "add_rmsnorm out")
    if residual.shape[1] != width:
        raise InvalidRequest("add_rmsnorm: width mismatch")
    if delta is not None:
        _need(delta, out.dtype, "add_rmsnorm delta", tuple(residual.shape))
    if rows is not None:
        _need(rows, torch.int32, "add_rmsnorm rows", (n_rows,))
    elif residual.shape[0] != n_rows:
        raise InvalidRequest("add_rmsnorm: row count mismatch")
    _check(library().mrs_add_rmsnorm(_is_bf16(out.dtype), residual.data_ptr(), _ptr(delta), weight.data_ptr(),
                                     float(eps), out.data_ptr(), _ptr(rows), n_rows, width, int(write_back),
                                     _stream()), "add_rmsnorm")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    width = x.shape[-1]
    _need(x, out.dtype, "rmsnorm input", tuple(out.shape))
    _need(weight, torch.float32, "rmsnorm weight", (width,))
    _need(out, None, "rmsnorm out")
    _check(library().mrs_rmsnorm(_is_bf16(x.dtype), x.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(),
                                 x.numel() // width, width, _stream()), "rmsnorm")


def rotation_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, d / 2, 2] float32: (cos, sin) of position * inv_freq, computed once a step for every layer that
    rotates by the same frequencies."""
    tokens, half = positions.shape[0], inv_freq.shape[0]
    _need(positions, torch.int32, "positions", (tokens,))
    _need(inv_freq, torch.float32, "inv_freq", (half,))
    out = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _check(library().mrs_rotation_table(positions.data_ptr(), inv_freq.data_ptr(), tokens, half, out.data_ptr(), _stream()),
           "rotation_table")
    return out


def qk_norm_rope_store(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                       v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
                       q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor | None, nq: int, nkv: int, d: int, page_size: int,
                       rotations: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotary of q and k, q to `q_out`, k and v into the paged cache
    ([pages, nkv, page_size, d]) at `slots`.  Without caches only q is produced.  `rotations`: the step's
    `rotation_table` for these positions and frequencies, if the caller has one; heads of 64, 128 and 256
    elements read their cosines and sines from it (and get one made here otherwise)."""
    tokens = qkv.shape[0]
    write_kv = k_cache is not None
    _need(qkv, None, "qkv", (tokens, (nq + 2 * nkv) * d))
    _need(q_out, qkv.dtype, "q_out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    if write_kv:
        _need(k_cache, qkv.dtype, "k cache")
        _need(v_cache, qkv.dtype, "v cache", tuple(k_cache.shape))
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d):
            raise InvalidRequest(f"cache shape {tuple(k_cache.shape)} does not match heads/page/head_dim")
        _need(slots, torch.int32, "slots", (tokens,))
    for w, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, name, (d,))
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", (d // 2,))
        if d in (64, 128, 256):
            if rotations is None:
                rotations = rotation_table(positions, inv_freq)
            _need(rotations, torch.float32, "rotations", (tokens, d // 2, 2))
        else:
            rotations = None
    else:
        rotations = None
    _check(library().mrs_qk_norm_rope_store(_is_bf16(qkv.dtype), qkv.data_ptr(), q_out.data_ptr(), _ptr(k_cache),
                                            _ptr(v_cache), positions.data_ptr(), _ptr(slots), _ptr(q_norm),
                                            _ptr(k_norm), float(eps), _ptr(inv_freq), _ptr(rotations), tokens, nq, nkv, d,
                                            page_size, int(write_kv), _stream()), "qk_norm_rope_store")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out = silu(gate) * up.  `gate_up` holds all gate columns and then all up columns (block 0), or
    alternating blocks of `block` gate columns and the `block` matching up columns."""
    tokens, inter = out.shape
    _need(gate_up, out.dtype, "gate_up", (tokens, 2 * inter))
    _need(out, None, "silu_mul out")
    if block < 0 or (block and inter % block):
        raise InvalidRequest("silu_mul: the width is no multiple of the block")
    _check(library().mrs_silu_mul(_is_bf16(out.dtype), gate_up.data_ptr(), out.data_ptr(), tokens, inter, int(block),
                                  _stream()), "silu_mul")


def attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, nq: int, nkv: int,
                   d: int, window: int = 0, scale: float | None = None) -> None:
    """Causal paged attention; one warp per (token, head); any sizes; float32 or bfloat16."""
    tokens = q.shape[0]
    _need(q, None, "q", (tokens, nq * d))
    _need(k_cache, q.dtype, "k cache")
    _need(v_cache, q.dtype, "v cache", tuple(k_cache.shape))
    _need(out, q.dtype, "attention out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(seq_of_token, torch.int32, "seq_of_token", (tokens,))
    _need(block_table, torch.int32, "block_table")
    page_size = k_cache.shape[2]
    if tuple(k_cache.shape[1:]) != (nkv, page_size, d):
        raise InvalidRequest("attention: cache shape does not match heads/head_dim")
    _check(library().mrs_attention_simt(_is_bf16(q.dtype), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                        out.data_ptr(), tokens, nq, nkv, d, page_size, block_table.shape[1],
                                        float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                        _stream()), "attention_simt")


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] . weight[N, K]^T in true float32 (CUDA-core FMA)."""
    m, k = x.shape
    n = weight.shape[0]
    _need(x, torch.float32, "gemm input")
    _need(weight, torch.float32, "gemm weight", (n, k))
    _need(out, torch.float32, "gemm out", (m, n))
    _check(library().mrs_gemm_f32(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, _stream()), "gemm_f32")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "argmax out", (rows,))
    _check(library().mrs_argmax(logits.data_ptr(), out.data_ptr(), rows, vocab, _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, draw_index: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature", (rows,))
    _need(top_k, torch.int32, "top_k", (rows,))
    _need(top_p, torch.float32, "top_p", (rows,))
    _need(seed, torch.int64, "seed", (rows,))
    _need(draw_index, torch.int32, "draw_index", (rows,))
    _need(out, torch.int32, "sample out", (rows,))
    _check(library().mrs_sample(logits.data_ptr(), rows, vocab, temperature.data_ptr(), top_k.data_ptr(),
                                top_p.data_ptr(), seed.data_ptr(), draw_index.data_ptr(), out.data_ptr(),
                                _stream()), "sample")


# ------------------------------------------------------------------------------------------------
# tensor-core attention, one library per head size
# ------------------------------------------------------------------------------------------------
_attention_libs: dict[int, ctypes.CDLL] = {}
_scratch: dict[torch.device, torch.Tensor] = {}

MMA_ROWS_WIDE, MMA_ROWS_NARROW = 64, 16


def attention_mma_supported(d: int, group: int) -> bool:
    return d % 16 == 0 and 16 <= d <= 256 and group <= MMA_ROWS_WIDE


def attention_mma_library(d: int) -> ctypes.CDLL:
    """The tensor-core attention compiled for head size `d` (built at first use)."""
    if d not in _attention_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_mma.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_mma_rows_mode.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_int, _c_int, _c_int,
                                                    _c_float, _c_int, _c_vp]
        lib.mrs_attention_mma_rows_mode.restype = _c_int
        lib.mrs_attention_mma_keys_mode.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_int, _c_int,
                                                    _c_int, _c_float, _c_int, _c_int, _c_vp]
        lib.mrs_attention_mma_keys_mode.restype = _c_int
        lib.mrs_attention_mma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_attention_mma_scratch_floats.restype = ctypes.c_longlong
        _attention_libs[d] = lib
    return _attention_libs[d]


_retired: list[torch.Tensor] = []     # outgrown scratch buffers: recorded steps may still point at them


def attention_scratch(device: torch.device, floats: int, lane: int = 0) -> torch.Tensor:
    """Scratch memory for split attention, kept and grown per device.  A buffer that is outgrown
    is never freed: a step recorded earlier replays with its address.  `lane`: the attention for few rows
    (0) and the one for prompt portions (1) have buffers of their own, because a step that holds both runs
    them side by side."""
    have = _scratch.get((device, lane))
    if have is None or have.numel() < floats:
        if have is not None:
            _retired.append(have)
        have = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _scratch[(device, lane)] = have
    return have


_side_streams: dict[torch.device, torch.cuda.Stream] = {}


def side_stream(device: torch.device) -> torch.cuda.Stream:
    """A second stream of the device, for kernels of one step that do not depend on one another."""
    if device not in _side_streams:
        _side_streams[device] = torch.cuda.Stream(device=device)
    return _side_streams[device]


_counters: dict[torch.device, torch.Tensor] = {}


def attention_counters(device: torch.device, count: int) -> torch.Tensor:
    """Zeroed ints by which the CTAs of a split attention find out which of them is last; the
    kernel leaves them zero.  Outgrown buffers stay alive like the scratch."""
    have = _counters.get(device)
    if have is None or have.numel() < count:
        if have is not None:
            _retired.append(have)
        have = torch.zeros(max(2 * count, 4096), dtype=torch.int32, device=device)
        _counters[device] = have
    return have


def _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d):
    tokens = q.shape[0]
    _need(q, torch.bfloat16, "q", (tokens, nq * d))
    _need(k_cache, torch.bfloat16, "k cache")
    _need(v_cache, torch.bfloat16, "v cache", tuple(k_cache.shape))
    _need(out, torch.bfloat16, "attention out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(block_table, torch.int32, "block_table")
    _need(tiles, torch.int32, "tiles")
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise InvalidRequest("attention tiles must be [n, 4] (sequence, first token, tokens, 0)")
    if tuple(k_cache.shape[1:]) != (nkv, k_cache.shape[2], d):
        raise InvalidRequest("attention: cache shape does not match heads/head_dim")


def attention_mma_rows(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                       window: int = 0, scale: float | None = None) -> None:
    """Tiles of up to 64 // (nq // nkv) tokens of one request each."""
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_mma_library(d)
    _check(lib.mrs_attention_mma_rows_mode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
                                           block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(),
                                           tiles.shape[0], out.data_ptr(), nq, nkv, k_cache.shape[2],
                                           float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                           _stream()), "attention_mma_rows")


def attention_mma_keys(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                       window: int = 0, splits: int = 1, scale: float | None = None,
                       scratch: torch.Tensor | None = None) -> None:
    """Tiles of up to 16 // (nq // nkv) tokens each; `splits` CTAs share the keys of a tile."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_mma_library(d)
    if splits > 1:
        need = lib.mrs_attention_mma_scratch_floats(tiles.shape[0], nkv, splits)
        if scratch is None:
            scratch = attention_scratch(q.device, need)
        _need(scratch, torch.float32, "attention scratch")
        if scratch.numel() < need:
            raise InvalidRequest(f"attention scratch holds {scratch.numel()} floats, {need} are needed")
        launch_count += 1          # the combine kernel
    _check(lib.mrs_attention_mma_keys_mode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
                                           block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(),
                                           tiles.shape[0], out.data_ptr(), _ptr(scratch) if splits > 1 else None,
                                           nq, nkv, k_cache.shape[2],
                                           float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                           int(splits), _stream()), "attention_mma_keys")


# ------------------------------------------------------------------------------------------------
# decode attention fed by bulk tensor copies (TMA), one library per head size (multiples of 64)
# ------------------------------------------------------------------------------------------------
_decode_libs: dict[int, ctypes.CDLL] = {}
_tensor_maps: dict[tuple, tuple] = {}


def attention_decode_tma_supported(d: int, group: int, page_size: int) -> bool:
    return d % 64 == 0 and 64 <= d <= 256 and group <= MMA_ROWS_NARROW and page_size >= 8


def attention_decode_tma_library(d: int) -> ctypes.CDLL:
    if d not in _decode_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_decode_tma.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_decode_tma_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_decode_tma_map.restype = _c_int
        lib.mrs_attention_decode_tma.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int,
                                                 _c_int, _c_float, _c_int, _c_int, _c_vp]
        lib.mrs_attention_decode_tma.restype = _c_int
        lib.mrs_attention_decode_tma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_attention_decode_tma_scratch_floats.restype = ctypes.c_longlong
        lib.mrs_attention_decode_tma_resident_clusters.argtypes = [_c_int]
        lib.mrs_attention_decode_tma_resident_clusters.restype = _c_int
        lib.mrs_attention_decode_tma_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_attention_decode_tma_take_error.restype = _c_int
        lib.mrs_attention_decode_tma_error_string.argtypes = [_c_int]
        lib.mrs_attention_decode_tma_error_string.restype = ctypes.c_char_p
        _decode_libs[d] = lib
        _register_error_word(f"attention_decode_tma (head size {d})", lib, "mrs_attention_decode_tma")
    return _decode_libs[d]


_resident_clusters: dict[tuple, int] = {}


def attention_decode_tma_resident_clusters(d: int, splits: int, device) -> int:
    """Thread-block clusters of `splits` CTAs of the decode attention (head size d) that the GPU holds at once, as
    the driver states it (B200, head size 128: 148, 71, 33 and 14 clusters of 2, 4, 8 and 16); 0 where no such
    cluster runs."""
    key = (d, splits, torch.device(device).index or 0)
    if key not in _resident_clusters:
        with torch.cuda.device(device):
            _resident_clusters[key] = int(attention_decode_tma_library(d).mrs_attention_decode_tma_resident_clusters(splits))
    return _resident_clusters[key]


def _aligned_block(size: int, alignment: int):
    """Host memory for a descriptor: (object that keeps it alive, aligned address)."""
    raw = ctypes.create_string_buffer(size + alignment)
    address = (ctypes.addressof(raw) + alignment - 1) // alignment * alignment
    return raw, address


def kv_tensor_map(cache: torch.Tensor) -> int:
    """Address of the tensor map of one layer's key or value pages [pages, kv_heads, page_size, d]
    (made once per tensor)."""
    key = (cache.data_ptr(), tuple(cache.shape))
    if key not in _tensor_maps:
        pages, nkv, page_size, d = cache.shape
        lib = attention_decode_tma_library(d)
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_attention_decode_tma_map(cache.data_ptr(), pages, nkv, page_size, address)
        if code != 0:
            raise BackendError(f"tensor map of the cache: {lib.mrs_attention_decode_tma_error_string(code).decode()}")
        _tensor_maps[key] = (keep, address)
    return _tensor_maps[key][1]


def attention_decode_tma(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                         window: int = 0, splits: int = 1, scale: float | None = None,
                         scratch: torch.Tensor | None = None) -> None:
    """Tiles of up to 16 // (nq // nkv) tokens each; keys and values come through bulk tensor copies."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_decode_tma_library(d)
    counters = None
    if splits > 1:
        need = lib.mrs_attention_decode_tma_scratch_floats(tiles.shape[0], nkv, splits)
        if scratch is None:
            scratch = attention_scratch(q.device, need)
        _need(scratch, torch.float32, "attention scratch")
        if scratch.numel() < need:
            raise InvalidRequest(f"attention scratch holds {scratch.numel()} floats, {need} are needed")
        counters = attention_counters(q.device, tiles.shape[0] * nkv)
    code = lib.mrs_attention_decode_tma(kv_tensor_map(k_cache), kv_tensor_map(v_cache), q.data_ptr(), positions.data_ptr(),
                                        block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(), tiles.shape[0],
                                        out.data_ptr(), _ptr(scratch) if splits > 1 else None, _ptr(counters), nq, nkv,
                                        k_cache.shape[2],
                                        float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                        int(splits), _stream())
    launch_count += 1
    if code != 0:
        raise BackendError(f"attention_decode_tma: {lib.mrs_attention_decode_tma_error_string(code).decode()} (code {code})")


# ------------------------------------------------------------------------------------------------
# tcgen05 attention for prompt portions, one library per head size (64, 128)
# ------------------------------------------------------------------------------------------------
_prefill_libs: dict[int, ctypes.CDLL] = {}
_prefill_kv_maps: dict[tuple, tuple] = {}
_prefill_q_map: dict[torch.device, tuple] = {}
PREFILL_TC_ROWS = 256          # two tiles of 128 query rows a CTA
PREFILL_TC_TILES = 2           # a tile holds 128 // group tokens (a group that does not divide 128 leaves rows empty)


def attention_prefill_tc_supported(d: int, group: int, page_size: int) -> bool:
    return d in (64, 128) and 1 <= group <= PREFILL_TC_ROWS // PREFILL_TC_TILES and page_size >= 8


def attention_prefill_tc_key_block(d: int) -> int:
    """Keys of one block of the tcgen05 kernel for prompt portions (the unit of its shares of a long context)."""
    lib = attention_prefill_tc_library(d)
    lib.mrs_attention_prefill_tc_key_block.restype = _c_int
    return lib.mrs_attention_prefill_tc_key_block()


def attention_prefill_tc_library(d: int) -> ctypes.CDLL:
    if d not in _prefill_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_prefill_tc.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_prefill_tc_kv_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_prefill_tc_q_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_prefill_tc.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_int, _c_int, _c_int, _c_float,
                                                 _c_int, _c_vp, _c_int, _c_vp]
        lib.mrs_attention_prefill_tc_partial_floats.argtypes = [_c_int, _c_int]
        lib.mrs_attention_prefill_tc_partial_floats.restype = ctypes.c_longlong
        for name in ("mrs_attention_prefill_tc_kv_map", "mrs_attention_prefill_tc_q_map", "mrs_attention_prefill_tc"):
            getattr(lib, name).restype = _c_int
        lib.mrs_attention_prefill_tc_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_attention_prefill_tc_take_error.restype = _c_int
        lib.mrs_attention_prefill_tc_error_string.argtypes = [_c_int]
        lib.mrs_attention_prefill_tc_error_string.restype = ctypes.c_char_p
        lib.mrs_attention_prefill_tc_rows.restype = _c_int
        if lib.mrs_attention_prefill_tc_rows() != PREFILL_TC_ROWS:
            raise BackendError(f"attention_prefill_tc takes {lib.mrs_attention_prefill_tc_rows()} rows a CTA, the planner expects {PREFILL_TC_ROWS}")
        _prefill_libs[d] = lib
        _register_error_word(f"attention_prefill_tc (head size {d})", lib, "mrs_attention_prefill_tc")
    return _prefill_libs[d]


def attention_prefill_tc(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                         window: int = 0, scale: float | None = None, shares: bool = False) -> None:
    """Work entries of up to 256 // (nq // nkv) tokens of one request each, on the tcgen05 tensor cores.  The
    fourth number of an entry is 0, or index | count << 8 when `count` entries (one after the other in the list)
    walk one share of the keys each (`shares` says that the list has such entries, whose sums a second kernel
    merges), or gap << 16 when the entry's second tile of 128 // (nq // nkv) tokens starts `gap` tokens behind
    the end of its first (the entry's token count is that of both tiles)."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_prefill_tc_library(d)

    def fail(code, what):
        raise BackendError(f"{what}: {lib.mrs_attention_prefill_tc_error_string(code).decode()} (code {code})")

    maps = []
    for cache in (k_cache, v_cache):
        key = (cache.data_ptr(), tuple(cache.shape))
        if key not in _prefill_kv_maps:
            keep, address = _aligned_block(128, 64)
            code = lib.mrs_attention_prefill_tc_kv_map(cache.data_ptr(), cache.shape[0], nkv, cache.shape[2], address)
            if code != 0:
                fail(code, "tensor map of the cache")
            _prefill_kv_maps[key] = (keep, address)
        maps.append(_prefill_kv_maps[key][1])
    if q.device not in _prefill_q_map:
        _prefill_q_map[q.device] = _aligned_block(128, 64)
    q_map = _prefill_q_map[q.device][1]
    code = lib.mrs_attention_prefill_tc_q_map(q.data_ptr(), q.shape[0], nq, nq // nkv, q_map)
    if code != 0:
        fail(code, "tensor map of the queries")
    launch_count += 2 if shares else 1
    partials = attention_scratch(q.device, lib.mrs_attention_prefill_tc_partial_floats(tiles.shape[0], nkv), lane=1) if shares else None
    code = lib.mrs_attention_prefill_tc(q_map, maps[0], maps[1], positions.data_ptr(), block_table.data_ptr(),
                                        block_table.shape[1], tiles.data_ptr(), tiles.shape[0], out.data_ptr(), nq, nkv,
                                        k_cache.shape[2], float(scale if scale is not None else 1.0 / math.sqrt(d)),
                                        int(window), _ptr(partials), int(shares), _stream())
    if code != 0:
        fail(code, "attention_prefill_tc")


# ------------------------------------------------------------------------------------------------
# tcgen05 matrix product for few rows (decoded tokens, short portions)
# ------------------------------------------------------------------------------------------------
_gemm_lib = None
_weight_maps: dict[tuple, tuple] = {}
_gemm_state: dict[torch.device, dict] = {}
GEMM_TC_MAX_ROWS = 128          # what the kernel takes
# Measured in the engine (decode steps at a context of 4,096, with the norms riding on the products), this kernel against
# the library's products: batch 8 9% faster; batch 16 5.13 against 5.22 ms a step at the 8B shape, 8.83 against 8.94 ms
# at the 14B shape (context 8,192), 2.36 against 2.46 ms at the 0.6B shape; batch 32 8.15 against 6.65 ms.  Its epilogue
# (a thread a weight row, looping over the rows) and the partial sums of the ranges of K grow with the rows.
GEMM_TC_BEST_ROWS = int(os.environ.get("MRS_GEMM_TC_BEST_ROWS", "16"))      # the variable: for measuring other crossovers


def gemm_tc_library() -> ctypes.CDLL:
    global _gemm_lib
    if _gemm_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("gemm_tc.cu", {})
        lib.mrs_gemm_tc_map.argtypes = [_c_vp, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_vp]
        lib.mrs_gemm_tc_map.restype = _c_int
        lib.mrs_gemm_tc_splits.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_gemm_tc_splits.restype = _c_int
        lib.mrs_gemm_tc_partial_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_gemm_tc_partial_floats.restype = ctypes.c_longlong
        lib.mrs_gemm_tc_counters.argtypes = [_c_int]
        lib.mrs_gemm_tc_counters.restype = _c_int
        lib.mrs_gemm_tc_small_m.argtypes = [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_vp, _c_vp]
        lib.mrs_gemm_tc_small_m.restype = _c_int
        lib.mrs_gemm_tc_qkv_heads.argtypes = [_c_vp] * 10 + [_c_float, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_int,
                                              _c_int, _c_int, _c_int, _c_vp, _c_vp]
        lib.mrs_gemm_tc_qkv_heads.restype = _c_int
        lib.mrs_gemm_tc_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_gemm_tc_take_error.restype = _c_int
        lib.mrs_gemm_tc_error_string.argtypes = [_c_int]
        lib.mrs_gemm_tc_error_string.restype = ctypes.c_char_p
        _gemm_lib = lib
        _register_error_word("gemm_tc", lib, "mrs_gemm_tc")
    return _gemm_lib


def gemm_tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Few rows, bfloat16, rows of a multiple of 8 elements on 16-byte boundaries: what the bulk
    tensor copies need."""
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and 0 < x.shape[0] <= GEMM_TC_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _gemm_device_state(device: torch.device) -> dict:
    state = _gemm_state.get(device)
    if state is None:
        state = {"sms": sm_count(device),
                 "counters": torch.zeros(4096, dtype=torch.int32, device=device),
                 "partials": torch.empty(1 << 24, dtype=torch.float32, device=device),
                 "x_map": _aligned_block(128, 64)}
        _gemm_state[device] = state
    return state


class _NormLink(ctypes.Structure):
    """The product's ties to the norms around it (`NormLink` of csrc/kernels/gemm_tc.cu)."""

    _fields_ = [("in_square_sums", _c_vp), ("in_parts", _c_int), ("in_stride", _c_int), ("in_inv_width", _c_float),
                ("in_eps", _c_float), ("stream", _c_vp), ("next_weight", _c_vp), ("out_square_sums", _c_vp)]


def _gemm_tc_prepare(x: torch.Tensor, weight: torch.Tensor, splits: int | None, max_mpad: int = 128):
    """Tensor maps, ranges of K and scratch for a product x . weight^T; returns (lib, state, w_map, x_map, splits, mpad)."""
    m, k = x.shape
    n = weight.shape[0]
    lib = gemm_tc_library()
    state = _gemm_device_state(x.device)
    key = (weight.data_ptr(), n, k)
    if key not in _weight_maps:
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_gemm_tc_map(weight.data_ptr(), n, k, 128, address)
        if code != 0:
            _gemm_fail(lib, code, "tensor map of a weight")
        _weight_maps[key] = (keep, address, lib.mrs_gemm_tc_splits(n, k, state["sms"]))
    _, w_map, planned = _weight_maps[key]
    splits = planned if splits is None else int(splits)      # another count only for measurements and tests
    mpad = 16 if m <= 16 else (32 if m <= 32 else (64 if m <= 64 else 128))
    if mpad > max_mpad:
        raise InvalidRequest(f"this product takes at most {max_mpad} rows, got {m}")
    x_map = state["x_map"][1]
    code = lib.mrs_gemm_tc_map(x.data_ptr(), m, k, mpad, x_map)
    if code != 0:
        _gemm_fail(lib, code, "tensor map of the activations")
    if splits > 1:
        need = lib.mrs_gemm_tc_partial_floats(m, n, splits)
        if state["partials"].numel() < need:       # outgrown buffers stay alive: recorded steps hold their addresses
            _retired.append(state["partials"])
            state["partials"] = torch.empty(2 * int(need), dtype=torch.float32, device=x.device)
        tiles = lib.mrs_gemm_tc_counters(n)
        if state["counters"].numel() < tiles:
            _retired.append(state["counters"])
            state["counters"] = torch.zeros(2 * tiles, dtype=torch.int32, device=x.device)
    return lib, state, w_map, x_map, splits, mpad


def _gemm_fail(lib, code, what):
    raise BackendError(f"{what}: {lib.mrs_gemm_tc_error_string(code).decode()} (code {code})")


def _norm_link(m: int, row_sums, stream=None, next_weight=None, out_sums=None):
    """The link structure of a product (or None): `row_sums` = (parts of the rows' sums of squares [parts, stride],
    the norm's width, its eps) of activations that are still to be divided by their root mean square."""
    if row_sums is None and stream is None:
        return None
    link = _NormLink()
    if row_sums is not None:
        sums, width, eps = row_sums
        _need(sums, torch.float32, "sums of squares")
        if sums.dim() != 2 or sums.shape[1] < m:
            raise InvalidRequest(f"sums of squares {tuple(sums.shape)} do not cover {m} rows")
        link.in_square_sums, link.in_parts, link.in_stride = sums.data_ptr(), sums.shape[0], sums.shape[1]
        link.in_inv_width, link.in_eps = 1.0 / float(width), float(eps)
    if stream is not None:
        link.stream, link.next_weight, link.out_square_sums = stream.data_ptr(), next_weight.data_ptr(), out_sums.data_ptr()
    return link


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
            splits: int | None = None, row_sums: tuple | None = None, residual: tuple | None = None) -> torch.Tensor | None:
    """out[M, N] = x[M, K] . weight[N, K]^T for M <= 128; bfloat16 in, float32 sums, `out` bfloat16 or float32.
    With `gated`, `weight` holds, in every block of 128 rows, 64 gate rows and then the 64 matching up rows, and
    out[M, N / 2] = silu(x . gate^T) * (x . up^T) in bfloat16.

    The RMSNorms around a product can ride on it.  `row_sums` = (parts [P, >= M] float32, width, eps): x holds
    rows that were multiplied by a norm's weights but not yet divided by their root mean square; the product
    multiplies row i's sums by rsqrt(sum_p parts[p, i] / width + eps).  `residual` = (stream [M, N] float32,
    next_weight [N] float32), up to 32 rows: stream += bfloat16(x . weight^T), out = bfloat16(stream *
    next_weight), and the parts of the new rows' sums of squares are returned ([ceil(N / 128), 16 or 32])."""
    m, k = x.shape
    n = weight.shape[0]
    _need(x, torch.bfloat16, "gemm input")
    _need(weight, torch.bfloat16, "gemm weight", (n, k))
    if gated:
        if n % 128:
            raise InvalidRequest("a gated product needs whole blocks of 64 gate and 64 up rows")
        _need(out, torch.bfloat16, "gemm out", (m, n // 2))
    else:
        _need(out, None, "gemm out", (m, n))
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise InvalidRequest("gemm out must be bfloat16 or float32")
    if m > GEMM_TC_MAX_ROWS:
        raise InvalidRequest(f"gemm_tc takes at most {GEMM_TC_MAX_ROWS} rows, got {m}")
    lib, state, w_map, x_map, splits, mpad = _gemm_tc_prepare(x, weight, splits, 32 if residual is not None else 128)
    out_sums = None
    if residual is not None:
        stream, next_weight = residual
        if gated or out.dtype is not torch.bfloat16:
            raise InvalidRequest("the product that adds to the stream is plain and writes bfloat16")
        _need(stream, torch.float32, "stream", (m, n))
        _need(next_weight, torch.float32, "next norm's weight", (n,))
        out_sums = torch.empty(((n + 127) // 128, mpad), dtype=torch.float32, device=x.device)
        link = _norm_link(m, row_sums, stream, next_weight, out_sums)
    else:
        link = _norm_link(m, row_sums)
    global launch_count
    launch_count += 1
    code = lib.mrs_gemm_tc_small_m(w_map, x_map, out.data_ptr(), int(out.dtype is torch.float32), int(gated),
                                   state["partials"].data_ptr(), state["counters"].data_ptr(), m, n, k, splits, mpad,
                                   state["sms"], ctypes.byref(link) if link is not None else None, _stream())
    if code != 0:
        _gemm_fail(lib, code, "gemm_tc")
    return out_sums


_qkv_heads_limits: tuple[int, int] | None = None


def gemm_tc_qkv_heads_limits() -> tuple[int, int]:
    """(head size, most rows) of the fused q/k/v projection, as its library states them."""
    global _qkv_heads_limits
    if _qkv_heads_limits is None:
        lib = gemm_tc_library()
        lib.mrs_gemm_tc_qkv_head_dim.restype = lib.mrs_gemm_tc_qkv_max_rows.restype = _c_int
        _qkv_heads_limits = (lib.mrs_gemm_tc_qkv_head_dim(), lib.mrs_gemm_tc_qkv_max_rows())
    return _qkv_heads_limits


def gemm_tc_qkv_heads_supported(x: torch.Tensor, weight: torch.Tensor, head_dim: int) -> bool:
    """Whether the fused q/k/v projection (head norms, rotation and cache write in the product's epilogue) takes
    these rows: the head size that the library's tiles are made for, few enough rows, and what `gemm_tc` needs."""
    if not gemm_tc_supported(x, weight):
        return False
    d, rows = gemm_tc_qkv_heads_limits()
    return head_dim == d and x.shape[0] <= rows


def gemm_tc_qkv_heads(x: torch.Tensor, weight: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                      v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
                      q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                      inv_freq: torch.Tensor | None, nq: int, nkv: int, row_sums: tuple | None = None) -> None:
    """The fused q/k/v projection for up to 32 rows and heads of 128 elements, with the per-head norms, the
    rotation and the cache write in the product's epilogue (what `qk_norm_rope_store` does after a product).
    `row_sums`: as for `gemm_tc`."""
    m, k = x.shape
    d, most = gemm_tc_qkv_heads_limits()
    _need(x, torch.bfloat16, "qkv input")
    _need(weight, torch.bfloat16, "qkv weight", ((nq + 2 * nkv) * d, k))
    _need(q_out, torch.bfloat16, "q_out", (m, nq * d))
    _need(positions, torch.int32, "positions", (m,))
    if m > most:
        raise InvalidRequest(f"the fused projection takes at most {most} rows, got {m}")
    page_size = 1
    if slots is not None:
        _need(slots, torch.int32, "slots", (m,))
        _need(k_cache, torch.bfloat16, "k cache")
        _need(v_cache, torch.bfloat16, "v cache", tuple(k_cache.shape))
        if tuple(k_cache.shape[1:]) != (nkv, k_cache.shape[2], d):
            raise InvalidRequest(f"cache shape {tuple(k_cache.shape)} does not match heads/head_dim")
        page_size = k_cache.shape[2]
    for w, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, name, (d,))
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", (d // 2,))
    lib, state, w_map, x_map, splits, mpad = _gemm_tc_prepare(x, weight, None, most)
    link = _norm_link(m, row_sums)
    global launch_count
    launch_count += 1
    code = lib.mrs_gemm_tc_qkv_heads(w_map, x_map, q_out.data_ptr(), _ptr(k_cache) if slots is not None else None,
                                     _ptr(v_cache) if slots is not None else None, positions.data_ptr(), _ptr(slots),
                                     _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), float(eps), nq, nkv, page_size,
                                     state["partials"].data_ptr(), state["counters"].data_ptr(), m, k, splits, mpad,
                                     state["sms"], ctypes.byref(link) if link is not None else None, _stream())
    if code != 0:
        _gemm_fail(lib, code, "gemm_tc_qkv_heads")


# ------------------------------------------------------------------------------------------------
# the tcgen05 gate/up product for many rows (prompt portions) with the activation in its epilogue
# ------------------------------------------------------------------------------------------------
_many_rows_lib = None
_many_rows_maps: dict[tuple, tuple] = {}
# Measured against the library's product followed by `silu_mul` (8B shape, K 4096, N 24576): 290 against 299 us at
# 2,048 rows, 418 against 429 us at 3,072, 550 against 646 us at 4,096; below 2,048 rows the library's pair is ahead
# (1,536: 221 against 217 us; 512: 90 against 83 us: the 128 x 256 tiles fill the SMs' last round badly).  At other
# shapes the order differs (prefill of 2,048 tokens: 14B shape, K 5120, N 34816: 58.2 ms with this kernel against
# 57.7 ms; 0.6B shape, K 1024, N 6144: 4.9 against 4.4 ms), so from GEMM_GATED_ROWS_MIN rows on the two are timed
# once per (N, K, thousand of rows) on the first such product and the faster one is kept (`gemm_gated_rows_wins`).
GEMM_GATED_ROWS_MIN = int(os.environ.get("MRS_GEMM_GATED_ROWS_MIN", "2048"))      # the variable: for measuring other crossovers
GEMM_GATED_MEASURE = "MRS_GEMM_GATED_ROWS_MIN" not in os.environ                  # False: the kernel from that many rows on
_gated_rows_choice: dict[tuple, bool] = {}


def gemm_gated_rows_wins(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 gate/up product with the activation in it is the faster way for these sizes on this
    device: at least GEMM_GATED_ROWS_MIN rows, and ahead of the library's product followed by `silu_mul` when the
    two were timed (three runs each after one, CUDA events, on buffers of their own; never while a step is being
    recorded: such steps have fewer rows anyway)."""
    rows = x.shape[0]
    if rows < GEMM_GATED_ROWS_MIN or not gemm_gated_rows_supported(x, weight):
        return False
    if not GEMM_GATED_MEASURE:
        return True
    n, k = weight.shape
    key = (x.device, n, k, 1 << (rows - 1).bit_length() if rows <= 1024 else 1024 * min(-(-rows // 1024), 16))
    if torch.cuda.is_current_stream_capturing():         # a step being recorded ran once just before: the choice is made
        return _gated_rows_choice.get(key, False)
    if key not in _gated_rows_choice:
        act = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=x.device)

        def own():
            gemm_gated_rows(x, weight, act)

        def library():
            silu_mul(torch.mm(x, weight.t()), act, 64)

        times = []
        for run in (own, library):
            run()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(3):
                run()
            end.record()
            end.synchronize()
            times.append(start.elapsed_time(end))
        _gated_rows_choice[key] = times[0] <= times[1]
    return _gated_rows_choice[key]


def gemm_many_rows_library() -> ctypes.CDLL:
    global _many_rows_lib
    if _many_rows_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("gemm_many_rows.cu", {})
        lib.mrs_gemm_many_rows_map.argtypes = [_c_vp, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_vp]
        lib.mrs_gemm_many_rows_map.restype = _c_int
        lib.mrs_gemm_gated_rows.argtypes = [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_vp]
        lib.mrs_gemm_gated_rows.restype = _c_int
        lib.mrs_gemm_many_rows_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_gemm_many_rows_take_error.restype = _c_int
        lib.mrs_gemm_many_rows_error_string.argtypes = [_c_int]
        lib.mrs_gemm_many_rows_error_string.restype = ctypes.c_char_p
        _many_rows_lib = lib
        _register_error_word("gemm_many_rows", lib, "mrs_gemm_many_rows")
    return _many_rows_lib


def _many_rows_maps_of(lib, x: torch.Tensor, weight: torch.Tensor):
    """(keep-alive of the activations' map, its address, the weights' map's address)."""
    n, k = weight.shape
    key = (weight.data_ptr(), n, k)
    if key not in _many_rows_maps:
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_gemm_many_rows_map(weight.data_ptr(), n, k, 256, address)
        if code != 0:
            raise BackendError(f"tensor map of a weight: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")
        _many_rows_maps[key] = (keep, address)
    x_keep, x_map = _aligned_block(128, 64)
    code = lib.mrs_gemm_many_rows_map(x.data_ptr(), x.shape[0], k, 128, x_map)
    if code != 0:
        raise BackendError(f"tensor map of the activations: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")
    return x_keep, x_map, _many_rows_maps[key][1]


def gemm_gated_rows_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """bfloat16, rows of a multiple of 8 elements on 16-byte boundaries, whole blocks of 64 gate and 64 up rows."""
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and weight.shape[0] % 128 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_gated_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[T, N / 2] = silu(x . gate^T) * (x . up^T) in bfloat16 for any number of rows; `weight` [N, K] holds, in
    every block of 128 rows, 64 gate rows and then the 64 matching up rows (as the gated `gemm_tc`)."""
    global launch_count
    t, k = x.shape
    n = weight.shape[0]
    _need(x, torch.bfloat16, "gated product input")
    _need(weight, torch.bfloat16, "gated product weight", (n, k))
    _need(out, torch.bfloat16, "gated product out", (t, n // 2))
    if not gemm_gated_rows_supported(x, weight):
        raise InvalidRequest("the gated product needs K a multiple of 8, whole blocks of 64 gate and 64 up rows and 16-byte alignment")
    lib = gemm_many_rows_library()
    x_keep, x_map, w_map = _many_rows_maps_of(lib, x, weight)
    launch_count += 1
    code = lib.mrs_gemm_gated_rows(x_map, w_map, out.data_ptr(), t, n, k, sm_count(x.device), _stream())
    del x_keep
    if code != 0:
        raise BackendError(f"gemm_gated_rows: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")


def wait_probe(limit_cycles: int = 1 << 16, device=None) -> bool:
    """Runs a one-warp kernel whose only act is a bounded wait on a barrier at which nobody arrives, with a limit
    of `limit_cycles` clocks (at most 2^24: milliseconds).  The wait gives up as every wait of the engine's
    kernels does when its time runs out: it raises the error word of its library and the kernel returns.
    Returns whether the wait gave up (it always does).  For the tests of the error path: `check_device_errors`
    raises afterwards, and the device is as usable as before."""
    lib = gemm_tc_library()
    lib.mrs_gemm_tc_wait_probe.argtypes = [ctypes.c_longlong, _c_vp, _c_vp]
    lib.mrs_gemm_tc_wait_probe.restype = _c_int
    flag = torch.zeros(1, dtype=torch.int32, device=device or torch.device("cuda", torch.cuda.current_device()))
    code = lib.mrs_gemm_tc_wait_probe(int(limit_cycles), flag.data_ptr(), _stream())
    if code != 0:
        _gemm_fail(lib, code, "wait_probe")
    torch.cuda.current_stream().synchronize()
    return bool(flag.item())


# ------------------------------------------------------------------------------------------------
# error words of the kernels that wait on barriers
# ------------------------------------------------------------------------------------------------
_mirror_view = None
_mirror = None          # pinned host words, one per library, that the kernels' error words are mirrored into


def _register_error_word(what: str, lib, prefix: str) -> None:
    """Keeps the library's reader and points its mirror at the next free pinned word."""
    global _mirror, _mirror_view
    if _mirror is None:
        _mirror = torch.zeros(16, dtype=torch.int32).pin_memory()
        _mirror_view = _mirror.numpy()
    index = len(_error_readers)
    reader = getattr(lib, f"{prefix}_take_error")
    _error_readers.append((what, reader))
    mirror = getattr(lib, f"{prefix}_mirror_errors")
    mirror.argtypes = [_c_vp]
    mirror.restype = _c_int
    if index < _mirror.numel():
        code = mirror(_mirror.data_ptr() + 4 * index)
        if code != 0:
            raise BackendError(f"{what}: cannot mirror the error word (CUDA error {code})")


def check_device_errors(certain: bool = False) -> None:
    """Raises when a kernel gave up a wait.  Called after a step, when the device is idle: the
    kernels mirror their error words into pinned host memory, so all is well as long as those
    words are zero; only then (or when `certain`) the words are read from the device and cleared."""
    if _mirror is not None and not certain and len(_error_readers) <= _mirror.numel() and not _mirror_view.any():
        return
    if _mirror is not None:
        _mirror.zero_()
    failed = []
    for what, reader in _error_readers:       # every word is read, and with that cleared
        word = ctypes.c_uint(0)
        code = reader(ctypes.byref(word))
        if code != 0:
            raise BackendError(f"{what}: reading the error word failed (CUDA error {code})")
        if word.value:
            failed.append(f"{what}: a kernel gave up waiting (error word {word.value:#x})")
    if failed:
        # a kernel that gave up may have left the arrival counters of its splits half counted: the next launch
        # that shares them must find zeros
        for counters in list(_counters.values()) + [state["counters"] for state in _gemm_state.values()]:
            counters.zero_()
        raise BackendError("; ".join(failed) + "; the step's result is invalid")
