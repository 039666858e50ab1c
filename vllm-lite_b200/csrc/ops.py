"""Python face of the CUDA kernels: one function per exported entry point.

Tensors are torch CUDA tensors used as plain device buffers; the kernels run on
torch's current stream.  Arguments are checked here (dtype, contiguity, sizes)
so that a kernel never sees a pointer that does not match its shape arguments.
A non-zero return code of an entry point raises `KernelError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {-2: "a size this kernel does not take", -3: "inconsistent arguments",
           -4: "the problem does not fit the built-in scratch memory"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, got {dtype}") from None


_SIGNATURES = {
    ("embed_norm", "vl_embed"): [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    ("embed_norm", "vl_rmsnorm_add"): [c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                       c_float, c_float, c_void_p],
    ("embed_norm", "vl_add_rmsnorm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    ("embed_norm", "vl_add_bias"): [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
    ("embed_norm", "vl_cast"): [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
    ("rope_cache", "vl_qk_norm_rope_write"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_int,
                                              c_void_p, c_void_p],
    ("attention", "vl_paged_attention"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p,
                                          c_void_p, c_void_p],
    ("rope_cache", "vl_head_norm_write"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                                           c_float, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
                                           c_int, c_void_p, c_void_p],
    ("latent", "vl_rope_heads"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("activation", "vl_sigmoid_gate"): [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("recurrent", "vl_token_shift_multi"): [c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_void_p],
    ("recurrent", "vl_decay_scan"): [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                     c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                     c_int, c_int, c_void_p],
    ("recurrent", "vl_decay_from_raw"): [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    ("rope_cache", "vl_conv_rows_norm_rope_write"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                                     c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                     c_int, c_int, c_int, c_longlong, c_void_p, c_void_p],
    ("rope_cache", "vl_rows_norm_rope_write"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_longlong, c_void_p, c_void_p],
    ("recurrent", "vl_token_shift"): [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_void_p],
    ("activation", "vl_unary_act"): [c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p],
    ("attention", "vl_decode_attention"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("attention", "vl_decode_attention_merge"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_prefill"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                         c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p],
    ("flash_tc5", "vl_flash_prefill_tc5"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p,
                                            c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_decode"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p],
    ("flash_attn", "vl_flash_decode_fused"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                              c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p],
    ("flash_decode_tma", "vl_flash_decode_tma"): [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    ("activation", "vl_silu_mul"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("activation", "vl_gated_act"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p,
                                     c_void_p],
    ("activation", "vl_scaled_sum"): [c_void_p, c_float, c_void_p, c_float, c_void_p, c_int, c_longlong, c_void_p],
    ("activation", "vl_scale_softcap"): [c_void_p, c_longlong, c_float, c_float, c_void_p],
    ("embed_norm", "vl_layernorm_add"): [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("embed_norm", "vl_layernorm_rows"): [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    ("latent", "vl_latent_norm_write"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                         c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("gemm_batched", "vl_gemm_batched_nt"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_longlong, c_longlong, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p],
    ("gemm_batched", "vl_gemm_grouped_fused"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                c_longlong, c_int, c_void_p, c_int, c_void_p, c_int, c_float, c_float, c_float,
                                                c_void_p],
    ("moe", "vl_moe_route"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float,
                              c_void_p, c_void_p, c_void_p],
    ("gemm_batched", "vl_gemm_rows_f32w"): [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_tc5_grouped", "vl_gemm_bf16_tc5_grouped"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                       c_void_p, c_int, c_float, c_float, c_float, c_void_p, c_void_p],
    ("moe", "vl_moe_align"): [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    ("moe", "vl_moe_gather"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("moe", "vl_moe_combine"): [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ("gemm_f32", "vl_gemm_f32_nt"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_bf16", "vl_gemm_bf16_small_m"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_void_p, c_int, c_void_p],
    ("gemm_bf16", "vl_gemm_bf16_small_m_fused"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_int,
                                                  c_void_p, c_void_p, c_void_p, c_void_p],
    ("gemm_tc5", "vl_gemm_bf16_tc5"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p, c_int, c_void_p],
    ("gemm_tc5_pair", "vl_gemm_bf16_tc5_pair"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_void_p, c_int, c_void_p],
    ("memprobe", "vl_read_only"): [c_void_p, c_longlong, c_void_p, c_void_p],
    ("sampling", "vl_apply_penalties"): [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p],
    ("sampling", "vl_sample"): [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p],
    ("hyper", "vl_hc_step"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("hyper", "vl_dyt_rows"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    ("recurrent", "vl_short_conv"): [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong,
                                     c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    ("recurrent", "vl_ssd_scan"): [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("recurrent", "vl_mlstm_scan"): [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                     c_float, c_float, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                     c_void_p],
    ("recurrent", "vl_delta_scan"): [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                     c_float, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                     c_int, c_void_p],
    ("recurrent", "vl_gate_norm"): [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_void_p,
                                    c_int, c_int, c_int, c_void_p],
}
_functions = {}
launch_count = 0          # kernels of this library launched so far (graph replays add theirs)


_pdl = False              # whether launches carry the programmatic-dependent-launch attribute: off unless the
                          # engine turns it on for a step of few tokens (the paired tcgen05 product never has it)
_pdl_libs = {}


def set_pdl(on: bool):
    """Launch the kernels that follow with (or without) the attribute that lets a kernel start while
    the one before it in the stream drains.  Every library holds the switch for its own launches."""
    global _pdl
    on = bool(on)
    if on != _pdl:
        _pdl = on
        for setter in _pdl_libs.values():
            setter(int(on))


def _fn(lib: str, name: str, defines=None):
    key = (lib, name, build._variant(defines))
    f = _functions.get(key)
    if f is None:
        handle = build.load(lib, defines)
        if key[::2] not in _pdl_libs and hasattr(handle, "vl_set_pdl"):
            setter = handle.vl_set_pdl
            setter.argtypes, setter.restype = [c_int], None
            setter(int(_pdl))
            _pdl_libs[key[::2]] = setter
        f = getattr(handle, name)
        f.argtypes = _SIGNATURES[(lib, name)]
        f.restype = c_int
        _functions[key] = f
    return f


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, name: str):
    global launch_count
    if code == 0:
        launch_count += 1
        return
    if code < 0:
        raise KernelError(f"{name} refused its arguments: {_ERRORS.get(code, code)}")
    raise KernelError(f"{name}: CUDA error {code} at launch")


def _need(t, dtype, name, ndim=None):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; the engine has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got {tuple(t.shape)}")


# ---------------------------------------------------------------- embed / norm
def embed(ids, table, out, err, scale=1.0):
    """out[t, :] = table[ids[t], :] * scale as float32.  ids int32 [T]; out float32 [T, H]."""
    _need(ids, torch.int32, "ids", 1); _need(table, None, "table", 2); _need(out, torch.float32, "out", 2)
    T, (V, H) = ids.shape[0], table.shape
    if out.shape != (T, H):
        raise KernelError(f"out must be [{T}, {H}], got {tuple(out.shape)}")
    _check(_fn("embed_norm", "vl_embed")(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), T, H, V,
                                         float(scale), _ptr(err), _stream()), "vl_embed")
    return out


def add_rmsnorm(x, delta, weight, eps, out, rows=None):
    """x float32 [T, H] (+= delta when given and rows is None); out[r] = rmsnorm(x[row r] (+ delta)) * weight."""
    _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1); _need(out, None, "out", 2)
    H = x.shape[1]
    R = x.shape[0] if rows is None else rows.shape[0]
    if weight.shape[0] != H or out.shape != (R, H):
        raise KernelError(f"norm shapes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if delta is not None:
        _need(delta, out.dtype, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError(f"delta {tuple(delta.shape)} must match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    _check(_fn("embed_norm", "vl_add_rmsnorm")(_ptr(x), _ptr(delta), _ptr(rows), _ptr(weight), _ptr(out),
                                               dtype_code(out.dtype), R, H, float(eps), _stream()), "vl_add_rmsnorm")
    return out


def add_bias(y, bias):
    """y[r, c] += bias[c] in place; y float32 or bfloat16 [rows, cols], bias float32 [cols]."""
    _need(y, None, "y", 2); _need(bias, torch.float32, "bias", 1)
    if bias.shape[0] != y.shape[1]:
        raise KernelError(f"add_bias: bias has {bias.shape[0]} entries for rows of {y.shape[1]}")
    _check(_fn("embed_norm", "vl_add_bias")(_ptr(y), dtype_code(y.dtype), _ptr(bias), y.shape[0], y.shape[1], _stream()),
           "vl_add_bias")
    return y


def cast(src, out):
    _need(src, None, "src"); _need(out, None, "out")
    if src.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check(_fn("embed_norm", "vl_cast")(_ptr(src), dtype_code(src.dtype), _ptr(out), dtype_code(out.dtype),
                                        src.numel(), _stream()), "vl_cast")
    return out


# ---------------------------------------------------------------- rope + cache
def qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, eps, inv_freq, rotary_dim,
                       k_cache, v_cache, num_heads, num_kv_heads, head_dim, err):
    """In place on the q part of qkv [T, (nq + 2 nkv) hd]; k and v go to the cache
    [pages, nkv, page_size, hd] at `slots` (int32 [T]; negative: no write)."""
    _need(qkv, None, "qkv", 2); _need(positions, torch.int32, "positions", 1)
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or positions.shape[0] != T:
        raise KernelError(f"qkv {tuple(qkv.shape)} does not match heads {num_heads}+2*{num_kv_heads} x {head_dim}")
    page_size, num_slots = 1, 0
    if slots is not None:
        _need(slots, torch.int32, "slots", 1)
        _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
        if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
            raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, torch.float32, n, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{n} must have head_dim={head_dim} entries")
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _check(_fn("rope_cache", "vl_qk_norm_rope_write")(
        _ptr(qkv), dtype_code(qkv.dtype), _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), float(eps),
        _ptr(inv_freq), int(rotary_dim if inv_freq is not None else 0), _ptr(k_cache) if slots is not None else None,
        _ptr(v_cache) if slots is not None else None, T, num_heads, num_kv_heads, head_dim, page_size, num_slots,
        qkv.shape[1], _ptr(err), _stream()), "vl_qk_norm_rope_write")
    return qkv


def rows_norm_rope_write(qk, positions, slots, q_weight, k_weight, eps, inv_freq, rotary_dim, q_out,
                         k_cache, v_cache, num_heads, num_kv_heads, head_dim, err, padded_head_dim=None):
    """qk float32 [T, >= (nq + nkv) hd] = q | k.  v <- k as it is; q and k are divided by the root mean square of their
    WHOLE row part (all heads at once) and multiplied by q_weight [nq hd] / k_weight [nkv hd]; then the first
    `rotary_dim` features of every head turn by the position; q goes to q_out [T, nq hdp], k and v to the cache
    [pages, nkv, page_size, hdp] at `slots` (None or negative: no write).  hdp = `padded_head_dim` (default hd) is the
    head size of the outputs; the features from hd on are zeros."""
    _need(qk, torch.float32, "qk", 2); _need(positions, torch.int32, "positions", 1); _need(q_out, None, "q_out", 2)
    _need(q_weight, torch.float32, "q_weight", 1); _need(k_weight, torch.float32, "k_weight", 1)
    T = qk.shape[0]
    Cq, Ck = num_heads * head_dim, num_kv_heads * head_dim
    hdp = int(padded_head_dim or head_dim)
    if qk.shape[1] < Cq + Ck or positions.shape[0] != T or q_out.shape != (T, num_heads * hdp) or q_weight.shape[0] != Cq \
            or k_weight.shape[0] != Ck:
        raise KernelError(f"rows_norm_rope_write: qk {tuple(qk.shape)}, q_out {tuple(q_out.shape)}, heads {num_heads}+{num_kv_heads} x {head_dim}")
    page_size, num_slots = 1, 0
    if slots is not None:
        _need(slots, torch.int32, "slots", 1)
        _need(k_cache, q_out.dtype, "k_cache", 4); _need(v_cache, q_out.dtype, "v_cache", 4)
        if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != hdp:
            raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {hdp}")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _check(_fn("rope_cache", "vl_rows_norm_rope_write")(
        _ptr(qk), qk.shape[1], _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq),
        int(rotary_dim if inv_freq is not None else 0), _ptr(q_out), dtype_code(q_out.dtype),
        _ptr(k_cache) if slots is not None else None, _ptr(v_cache) if slots is not None else None, T, num_heads,
        num_kv_heads, head_dim, hdp, page_size, num_slots, _ptr(err), _stream()), "vl_rows_norm_rope_write")
    return q_out


_conv_rows_max = None


def conv_rows_fused_ok(channels) -> bool:
    """Whether `conv_rows_norm_rope_write` takes rows of this many q and k channels (it keeps one in shared memory)."""
    global _conv_rows_max
    if _conv_rows_max is None:
        _conv_rows_max = int(build.load("rope_cache").vl_conv_rows_max())
    return 0 < channels <= _conv_rows_max


def conv_rows_norm_rope_write(proj, weight, in_bias, state, state_off, cu, state_slots, req_index, longest, positions, slots,
                              q_weight, k_weight, eps, inv_freq, rotary_dim, q_out, k_cache, v_cache, num_heads, num_kv_heads,
                              head_dim, err, padded_head_dim=None):
    """`short_conv` (no activation, `in_bias` added to the rows as they are read) of the first (nq + nkv) hd columns of
    proj [T, ld] and `rows_norm_rope_write` of the result in one launch: the convolved row stays in shared memory.  The
    request's state row [(taps-1), C] at `state_off` is read by this launch and renewed by it when every request brings
    one token (`longest` == 1), else by the convolution's state pass that follows.  The same bits as the two in turn."""
    _need(proj, None, "proj", 2); _need(weight, torch.float32, "weight", 2); _need(positions, torch.int32, "positions", 1)
    _need(q_weight, torch.float32, "q_weight", 1); _need(k_weight, torch.float32, "k_weight", 1); _need(q_out, proj.dtype, "q_out", 2)
    _need(req_index, torch.int32, "req_index", 1)
    T = proj.shape[0]
    Cq, Ck = num_heads * head_dim, num_kv_heads * head_dim
    C, taps = Cq + Ck, weight.shape[1]
    hdp = int(padded_head_dim or head_dim)
    if proj.shape[1] < C or weight.shape[0] != C or positions.shape[0] != T or req_index.shape[0] != T \
            or q_out.shape != (T, num_heads * hdp) or q_weight.shape[0] != Cq or k_weight.shape[0] != Ck:
        raise KernelError(f"conv_rows_norm_rope_write: proj {tuple(proj.shape)}, q_out {tuple(q_out.shape)}, heads {num_heads}+{num_kv_heads} x {head_dim}")
    if in_bias is not None:
        _need(in_bias, torch.float32, "in_bias", 1)
        if in_bias.shape[0] != C:
            raise KernelError("conv_rows_norm_rope_write: in_bias has one entry per channel")
    page_size, num_slots = 1, 0
    if slots is not None:
        _need(slots, torch.int32, "slots", 1)
        _need(k_cache, q_out.dtype, "k_cache", 4); _need(v_cache, q_out.dtype, "v_cache", 4)
        if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != hdp:
            raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {hdp}")
        page_size = k_cache.shape[2]
        num_slots = k_cache.shape[0] * page_size
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("inv_freq must have rotary_dim / 2 entries")
    _seg_args(cu, state_slots)
    sp, stride = _state_args(state, state_off, max((taps - 1) * C, 1))
    longest = int(longest or max(T, 1))
    _check(_fn("rope_cache", "vl_conv_rows_norm_rope_write")(
        _ptr(proj), proj.shape[1], _ptr(weight), _ptr(in_bias), taps, sp, stride, _ptr(cu), _ptr(state_slots), _ptr(req_index),
        int(longest == 1), _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq),
        int(rotary_dim if inv_freq is not None else 0), _ptr(q_out), dtype_code(q_out.dtype),
        _ptr(k_cache) if slots is not None else None, _ptr(v_cache) if slots is not None else None, T, num_heads,
        num_kv_heads, head_dim, hdp, page_size, num_slots, _ptr(err), _stream()), "vl_conv_rows_norm_rope_write")
    if longest > 1 and taps > 1:
        short_conv(proj, 0, C, weight, None, state, state_off, cu, state_slots, None, act=False, longest=longest, in_bias=in_bias)
    return q_out


def token_shift(x, mu, state, state_off, cu, slots, req_index, positions, out):
    """out[t] = x[t] + (x[t - 1] - x[t]) * mu in float32, x float32 [T, W]; the row before a portion's first token is
    state[slot, state_off : state_off + W] (zeros in a fresh slot), which the launch replaces by the portion's last row."""
    _need(x, torch.float32, "x", 2); _need(mu, torch.float32, "mu", 1); _need(out, None, "out", 2)
    T, W = x.shape
    if mu.shape[0] != W or out.shape != (T, W) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("token_shift: shapes disagree")
    base, stride = _state_args(state, state_off, W)
    B = _seg_args(cu, slots)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _check(_fn("recurrent", "vl_token_shift")(_ptr(x), _ptr(mu), base, stride, _ptr(cu), _ptr(slots), _ptr(req_index),
                                              _ptr(positions), _ptr(out), dtype_code(out.dtype), T, W, _stream()),
           "vl_token_shift")
    return out


# ---------------------------------------------------------------- attention
def _check_sinks(sinks, num_heads):
    if sinks is not None:
        _need(sinks, torch.float32, "sinks", 1)
        if sinks.shape[0] != num_heads:
            raise KernelError(f"sinks must hold one number per query head ({num_heads}), got {sinks.shape[0]}")


WEIGHTINGS = {"softmax": 0, "sigmoid": 1}


def _check_variant(qkv, num_heads, weighting, chunk, head_bias, gate, sinks):
    """The options every attention entry point shares: `weighting` "softmax", or "sigmoid" (a visible key weighs
    sigmoid(score + head_bias[h]) by itself, nothing is divided by a sum; no sinks); `chunk`: positions in blocks of
    that many, a query reads no key of an earlier block; `gate` [T, >= nq] in the activation dtype (a view whose rows
    may be wider): head h's output for token t is multiplied by sigmoid(gate[t, h]).  Returns (mode, chunk, gate stride)."""
    if weighting not in WEIGHTINGS:
        raise KernelError(f"attention weighting {weighting!r}; known: {', '.join(WEIGHTINGS)}")
    if weighting == "sigmoid" and sinks is not None:
        raise KernelError("a sink belongs to a softmax")
    if head_bias is not None:
        _need(head_bias, torch.float32, "head_bias", 1)
        if weighting != "sigmoid" or head_bias.shape[0] != num_heads:
            raise KernelError("head_bias: one float32 number per query head, for the sigmoid weighting")
    stride = 0
    if gate is not None:
        if not gate.is_cuda or gate.dtype != qkv.dtype or gate.dim() != 2 or gate.shape[0] != qkv.shape[0] \
                or gate.shape[1] < num_heads or gate.stride(1) != 1:
            raise KernelError("gate must be [T, >= heads] in the activation dtype with unit stride along the heads")
        stride = gate.stride(0)
    if chunk is not None and chunk <= 0:
        raise KernelError(f"a chunk of {chunk} positions")
    return WEIGHTINGS[weighting], int(chunk or 0), stride


def _check_score_shape(num_heads, softcap, distance):
    """Two options on the scores that every attention entry point shares: `softcap` c > 0 bounds a score,
    s <- c tanh(s / c); `distance` (a, b), float32 [num_heads] each, then takes a[h] ln(1 + b[h] (i - j)) off the score of
    the key that lies i - j positions back.  Returns (cap or 0.0, a, b)."""
    cap = float(softcap or 0.0)
    if cap < 0:
        raise KernelError(f"a score cap of {cap}")
    if distance is None:
        return cap, None, None
    a, b = distance
    _need(a, torch.float32, "distance[0]", 1); _need(b, torch.float32, "distance[1]", 1)
    if a.shape[0] != num_heads or b.shape[0] != num_heads:
        raise KernelError(f"the distance bias has two numbers per query head ({num_heads})")
    return cap, a, b


def paged_attention(qkv, out, k_cache, v_cache, block_table, req_index, positions,
                    num_heads, num_kv_heads, head_dim, scale, window, err, sinks=None,
                    weighting="softmax", chunk=None, head_bias=None, gate=None, softcap=None, distance=None):
    """out [T, nq*hd] = attention of the q part of qkv over the pages of each token's request.
    `sinks` (float32 [nq]): one more term exp(sinks[h]) in every softmax denominator of head h.
    `weighting`, `chunk`, `head_bias`, `gate`: see `_check_variant`.  `softcap`, `distance`: see `_check_score_shape`."""
    _check_sinks(sinks, num_heads)
    cap, dist_a, dist_b = _check_score_shape(num_heads, softcap, distance)
    mode, chunk, gate_stride = _check_variant(qkv, num_heads, weighting, chunk, head_bias, gate, sinks)
    _need(qkv, None, "qkv", 2); _need(out, qkv.dtype, "out", 2)
    _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("paged_attention: token counts or widths disagree")
    if qkv.shape[1] < num_heads * head_dim:
        raise KernelError("paged_attention: qkv rows are narrower than the query heads")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
    _check(_fn("attention", "vl_paged_attention")(
        _ptr(qkv), qkv.shape[1], _ptr(out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(req_index), _ptr(positions),
        T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), _ptr(sinks), mode, chunk, _ptr(head_bias), _ptr(gate), gate_stride,
        cap, _ptr(dist_a), _ptr(dist_b), _ptr(err), _stream()), "vl_paged_attention")
    return out


DECODE_CHUNK = 256        # key positions per block of the split decode kernel


def decode_attention_scratch(num_tokens, num_heads, head_dim, max_context, chunk=DECODE_CHUNK):
    """(splits, floats of part_acc, floats of part_ml) that `decode_attention` needs."""
    S = max(1, -(-int(max_context) // chunk))
    return S, num_tokens * num_heads * S * head_dim, num_tokens * num_heads * S * 2


def decode_attention(qkv, out, k_cache, v_cache, block_table, req_index, positions, num_heads, num_kv_heads,
                     head_dim, scale, window, max_context, part_acc, part_ml, err, chunk=DECODE_CHUNK):
    """Same function as `paged_attention`, for steps of few tokens per request: the key range of
    a token is split over blocks of `chunk` positions and merged.  `max_context` bounds
    position + 1 of every token; part_acc / part_ml are float32 scratch (see
    `decode_attention_scratch`)."""
    _need(qkv, None, "qkv", 2); _need(out, qkv.dtype, "out", 2)
    _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _need(part_acc, torch.float32, "part_acc"); _need(part_ml, torch.float32, "part_ml")
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("decode_attention: token counts or widths disagree")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")
    S, need_acc, need_ml = decode_attention_scratch(T, num_heads, head_dim, max_context, chunk)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError(f"decode_attention: scratch too small ({part_acc.numel()} < {need_acc})")
    _check(_fn("attention", "vl_decode_attention")(
        _ptr(qkv), qkv.shape[1], _ptr(out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
        _ptr(block_table), block_table.shape[1], _ptr(req_index), _ptr(positions),
        T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), chunk, S, _ptr(part_acc), _ptr(part_ml), _ptr(err), _stream()),
        "vl_decode_attention")
    global launch_count
    launch_count += 1           # two kernels: the split pass and the merge
    return out


_max_clusters = {}


def flash_decode_max_cluster(head_dim) -> int:
    """Most chunks of a token that `vl_flash_decode` merges as the blocks of one cluster: 16 where the device
    takes clusters beyond the portable 8, else 8."""
    v = _max_clusters.get(head_dim)
    if v is None:
        fn = build.load("flash_attn", {"FA_HD": head_dim}).vl_flash_decode_max_cluster
        fn.restype = c_int
        v = _max_clusters[head_dim] = int(fn())
    return v


def decode_chunk_for(num_tokens, num_kv_heads, max_context, target_blocks=256, head_dim=None) -> int:
    """Key positions per block of the split decode kernels: the largest of 256..1024 that still
    gives most of the 148 SMs two blocks (a block's start-up is paid once per chunk; measured at
    batch 8, context 4,096: 4.80 / 4.55 / 4.38 ms a step with chunks of 256 / 512 / 1,024)."""
    ctx = int(max_context)
    for chunk in (1024, 512):
        if num_tokens * num_kv_heads * -(-ctx // chunk) >= target_blocks:
            return chunk
    # Too few blocks either way.  What bounds so few blocks is a warp's own pace (2,200 cycles for its 16
    # keys of every 64), so the shortest chunks win whose blocks still merge as one cluster per token (8
    # blocks, 16 where the device takes it) and have an SM each: one request at 4,096 keys, 16 chunks of 256
    # against 8 of 512: 3.24 -> 3.08 ms a step; two requests (256 blocks, two to an SM): 3.26 -> 3.43, so not there
    if head_dim is not None and flash_supported(torch.bfloat16, head_dim):
        most = flash_decode_max_cluster(head_dim)
        for chunk in (128, 256, 512, 1024):
            chunks = -(-ctx // chunk)
            if chunks <= most and num_tokens * num_kv_heads * chunks <= 2 * sm_pairs():
                return chunk
    return 512 if -(-ctx // 512) <= 8 else 256


def flash_supported(dtype, head_dim) -> bool:
    """The tensor-core attention kernels take bfloat16 and head sizes in steps of 16 up to 256."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim):
    _need(qkv, torch.bfloat16, "qkv", 2)
    _need(k_cache, torch.bfloat16, "k_cache", 4); _need(v_cache, torch.bfloat16, "v_cache", 4)
    _need(block_table, torch.int32, "block_table", 2)
    if qkv.shape[1] < num_heads * head_dim or qkv.shape[1] % 8:
        raise KernelError("flash attention: qkv rows are too narrow or not 16-byte aligned")
    if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise KernelError(f"cache {tuple(k_cache.shape)} does not match kv heads {num_kv_heads} x {head_dim}")


def flash_prefill(qkv, out, k_cache, v_cache, block_table, tiles, num_heads, num_kv_heads, head_dim, scale, window, err,
                  tile_rows=64, sinks=None, weighting="softmax", mask_chunk=None, head_bias=None, gate=None, softcap=None,
                  distance=None):
    """Tensor-core (mma.sync) attention for prompt portions.  `tiles` int32 [n, 4]: (row of the block
    table, index of the tile's first token in the step, tokens (<= tile_rows), position of the first
    token); the tiles of a step cover every token that the kernel is to serve once.
    `weighting`, `mask_chunk` (the `chunk` there), `head_bias`, `gate`: see `_check_variant`; `softcap`, `distance`: see
    `_check_score_shape`."""
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _check_sinks(sinks, num_heads)
    mode, mask_chunk, gate_stride = _check_variant(qkv, num_heads, weighting, mask_chunk, head_bias, gate, sinks)
    cap, dist_a, dist_b = _check_score_shape(num_heads, softcap, distance)
    _need(out, torch.bfloat16, "out", 2); _need(tiles, torch.int32, "tiles", 2)
    if out.shape != (qkv.shape[0], num_heads * head_dim) or tiles.shape[1] != 4:
        raise KernelError("flash_prefill: shapes disagree")
    _check(_fn("flash_attn", "vl_flash_prefill", {"FA_HD": head_dim})(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(tiles), tiles.shape[0], int(tile_rows), num_heads, num_kv_heads, head_dim, k_cache.shape[2],
        k_cache.shape[0], float(scale), int(window or 0), _ptr(err), _ptr(sinks), mode, mask_chunk, _ptr(head_bias),
        _ptr(gate), gate_stride, cap, _ptr(dist_a), _ptr(dist_b), _stream()), "vl_flash_prefill")
    return out


FLASH_TC5_TILE = 128


def flash_tc5_supported(dtype, head_dim, page_size) -> bool:
    """The tcgen05 attention kernel takes bfloat16, head sizes 64 and 128, and pages of a multiple of
    8 positions that divide 64 or are a multiple of it."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 8 == 0
            and (64 % page_size == 0 if page_size < 64 else page_size % 64 == 0))


def flash_prefill_tc5(qkv, out, k_cache, v_cache, block_table, tiles, num_heads, num_kv_heads, head_dim, scale, window, err,
                      sinks=None, weighting="softmax", mask_chunk=None, head_bias=None, gate=None, softcap=None, distance=None):
    """Attention for prompt portions on the tcgen05 tensor cores; `tiles` as for `flash_prefill`,
    up to 128 tokens each.  `weighting`, `mask_chunk` (the `chunk` there), `head_bias`, `gate`: see `_check_variant`;
    `softcap`, `distance`: see `_check_score_shape`."""
    cap, dist_a, dist_b = _check_score_shape(num_heads, softcap, distance)
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _need(out, torch.bfloat16, "out", 2); _need(tiles, torch.int32, "tiles", 2)
    _check_sinks(sinks, num_heads)
    mode, mask_chunk, gate_stride = _check_variant(qkv, num_heads, weighting, mask_chunk, head_bias, gate, sinks)
    if out.shape != (qkv.shape[0], num_heads * head_dim) or tiles.shape[1] != 4:
        raise KernelError("flash_prefill_tc5: shapes disagree")
    if not flash_tc5_supported(qkv.dtype, head_dim, k_cache.shape[2]):
        raise KernelError(f"flash_prefill_tc5: head size {head_dim} / page size {k_cache.shape[2]} not taken")
    _check(_fn("flash_tc5", "vl_flash_prefill_tc5", {"FA_HD": head_dim})(
        _ptr(qkv), qkv.shape[1], _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(tiles), tiles.shape[0], num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
        float(scale), int(window or 0), _ptr(err), _ptr(sinks), mode, mask_chunk, _ptr(head_bias), _ptr(gate), gate_stride,
        cap, _ptr(dist_a), _ptr(dist_b), _stream()), "vl_flash_prefill_tc5")
    return out


_merge_caps = {}


def _own_merge_cap(head_dim) -> int:
    """Most chunks per token that `vl_flash_decode` of this head size merges itself."""
    cap = _merge_caps.get(head_dim)
    if cap is None:
        cap = _merge_caps[head_dim] = int(build.load("flash_attn", {"FA_HD": head_dim}).vl_flash_decode_own_merge_cap())
    return cap


flash_decode_own_merge_cap = _own_merge_cap


def flash_decode_arrivals(num_tokens, num_heads, num_kv_heads) -> int:
    """Counters (int32) that `flash_decode` needs in `arrivals` for this many tokens."""
    return num_tokens * num_kv_heads * -(-(num_heads // num_kv_heads) // 16)


STREAM_DECODE_MIN_KEYS = 8 * 49152      # tokens x KV heads x context bound from which the persistent TMA kernel is used


def flash_decode_streams(dtype, num_tokens, num_kv_heads, head_dim, page_size, max_context) -> bool:
    """Whether `flash_decode` left to itself serves such a step with the persistent TMA kernel (else a block per chunk).
    Measured (Qwen3-8B heads, pages of 64): it wins from 64-position pages on (TMA boxes of 8 KB, not 2 KB) when
    the step streams enough keys to keep every SM's block busy: 16 tokens x 4,096 keys 55.8 us against 60.0 for a
    block per chunk, 64 x 4,096: 170 against 188, 8 x 16,384: 96 against 108; at 8 x 4,096 and below the block per
    chunk, which merges in the same launch, is level or ahead."""
    return (flash_tc5_supported(dtype, head_dim, page_size) and page_size >= 64
            and num_tokens * num_kv_heads * int(max_context) >= STREAM_DECODE_MIN_KEYS)


def flash_decode(qkv, out, k_cache, v_cache, block_table, req_index, positions, num_heads, num_kv_heads,
                 head_dim, scale, window, max_context, part_acc, part_ml, err, chunk=DECODE_CHUNK, token_index=None,
                 stream_kernel=None, arrivals=None, fold=None, sinks=None, weighting="softmax", mask_chunk=None,
                 head_bias=None, gate=None, softcap=None, distance=None):
    """Tensor-core version of `decode_attention` (bfloat16): every block takes a chunk of a token's
    keys; the chunks are merged by the block that finishes last (`arrivals`: int32 counters,
    `flash_decode_arrivals` of them, zero before the first call and left zero) or, without
    `arrivals`, by a second kernel.
    The split pass is the persistent TMA kernel where it takes the head size, pages hold at
    least 64 positions and the step reads STREAM_DECODE_MIN_KEYS keys or more (`stream_kernel`: None =
    that rule, True / False to force; it always merges with the second kernel), else a block per chunk.
    `token_index` (int32) restricts the launch to some tokens of the step (the others' rows of `out`
    are left alone); the scratch is then sized for that many tokens.
    `fold` = (q_weight, k_weight, eps, inv_freq, rotary_dim, slots) folds the step's `qk_norm_rope_write`
    into the block-per-chunk kernel (the TMA kernel does not take it): qkv then holds the rows as the
    projection left them, every token is the last of its request, and the token's key and value are
    written to the cache by this launch (slots None: not written).  The same bits as the two kernels in turn.
    `weighting`, `mask_chunk` (the `chunk` there), `head_bias`, `gate`: see `_check_variant`.  The sigmoid and the gate
    go with the block-per-chunk kernel that merges its chunks itself (`arrivals` given, few enough chunks).
    `softcap`, `distance` (see `_check_score_shape`) go with the block-per-chunk kernel, merged either way."""
    _flash_checks(qkv, k_cache, v_cache, block_table, num_heads, num_kv_heads, head_dim)
    _check_sinks(sinks, num_heads)
    mode, mask_chunk, gate_stride = _check_variant(qkv, num_heads, weighting, mask_chunk, head_bias, gate, sinks)
    cap, dist_a, dist_b = _check_score_shape(num_heads, softcap, distance)
    variant = bool(mode or mask_chunk or gate is not None)
    if (variant or cap or dist_a is not None) and fold is not None:
        raise KernelError("flash_decode: the folded head work goes with the plain softmax")
    if cap or dist_a is not None:
        if stream_kernel:
            raise KernelError("flash_decode: capped or biased scores go with the block-per-chunk kernel")
        stream_kernel = False
    if sinks is not None and fold is not None:
        raise KernelError("flash_decode: the folded head work and sinks do not go together")
    _need(out, torch.bfloat16, "out", 2)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _need(part_acc, torch.float32, "part_acc"); _need(part_ml, torch.float32, "part_ml")
    T = qkv.shape[0]
    if out.shape != (T, num_heads * head_dim) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("flash_decode: token counts or widths disagree")
    if token_index is not None:
        _need(token_index, torch.int32, "token_index", 1)
        T = token_index.shape[0]
    S, need_acc, need_ml = decode_attention_scratch(T, num_heads, head_dim, max_context, chunk)
    if part_acc.numel() < need_acc or part_ml.numel() < need_ml:
        raise KernelError(f"flash_decode: scratch too small ({part_acc.numel()} < {need_acc})")
    if variant:
        if stream_kernel or arrivals is None or S > _own_merge_cap(head_dim):
            raise KernelError("flash_decode: weighting, mask chunk and gate go with the kernel that merges its chunks itself")
        stream_kernel = False
    if stream_kernel is None:
        stream_kernel = fold is None and flash_decode_streams(qkv.dtype, T, num_kv_heads, head_dim, k_cache.shape[2], max_context)
    if fold is not None and (stream_kernel or token_index is not None):
        raise KernelError("flash_decode: the folded norm and rotation go with the block-per-chunk kernel and whole steps")
    args = (_ptr(qkv), qkv.shape[1], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(req_index), _ptr(positions), T, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
            float(scale), int(window or 0), chunk, S, _ptr(part_acc), _ptr(part_ml), _ptr(err), _ptr(token_index))
    if stream_kernel:
        _check(_fn("flash_decode_tma", "vl_flash_decode_tma", {"FA_HD": head_dim})(*args, _stream()), "vl_flash_decode_tma")
    else:
        if arrivals is not None and S > _own_merge_cap(head_dim):
            arrivals = None
        if arrivals is not None:
            _need(arrivals, torch.int32, "arrivals", 1)
            if arrivals.numel() < flash_decode_arrivals(T, num_heads, num_kv_heads):
                raise KernelError("flash_decode: too few arrival counters")
        if fold is None:
            _check(_fn("flash_attn", "vl_flash_decode", {"FA_HD": head_dim})(
                *args, _ptr(out) if arrivals is not None else None, _ptr(arrivals), _ptr(sinks), mode, mask_chunk,
                _ptr(head_bias), _ptr(gate), gate_stride, cap, _ptr(dist_a), _ptr(dist_b), _stream()), "vl_flash_decode")
        else:
            qw, kw, eps, inv_freq, rot, slots = fold
            for t, n in ((qw, "q_weight"), (kw, "k_weight"), (inv_freq, "inv_freq")):
                if t is not None:
                    _need(t, torch.float32, n, 1)
            if (qw is None) != (kw is None) or (qw is not None and (qw.shape[0] != head_dim or kw.shape[0] != head_dim)):
                raise KernelError("flash_decode: the head norm's weights do not match the head size")
            if inv_freq is not None and inv_freq.shape[0] * 2 != rot:
                raise KernelError("flash_decode: inv_freq does not match the rotary dimension")
            if slots is not None:
                _need(slots, torch.int32, "slots", 1)
                if slots.shape[0] < T:
                    raise KernelError("flash_decode: fewer slots than tokens")
            if qkv.shape[1] < (num_heads + 2 * num_kv_heads) * head_dim:
                raise KernelError("flash_decode: the rows do not hold q, k and v")
            _check(_fn("flash_attn", "vl_flash_decode_fused", {"FA_HD": head_dim})(
                *args, _ptr(out) if arrivals is not None else None, _ptr(arrivals),
                _ptr(qw), _ptr(kw), float(eps), _ptr(inv_freq), int(rot if inv_freq is not None else 0), _ptr(slots),
                _stream()), "vl_flash_decode_fused")
        if arrivals is not None:
            return out
    _check(_fn("attention", "vl_decode_attention_merge")(
        _ptr(part_acc), _ptr(part_ml), _ptr(positions), _ptr(out), dtype_code(out.dtype), T, num_heads, head_dim,
        chunk, S, int(window or 0), _ptr(token_index), _ptr(sinks), _stream()), "vl_decode_attention_merge")
    return out


# ---------------------------------------------------------------- feed-forward
SWIGLU_GROUP = 8          # gate/up interleave that the matrix-product kernels' fused activation expects


def silu_mul(gate_up, out, group=0):
    """out[t, i] = silu(gate_i) * up_i of gate_up [T, 2I].  group = 0: gate columns, then up columns;
    group = g: blocks of g gate columns followed by their g up columns."""
    _need(gate_up, None, "gate_up", 2); _need(out, gate_up.dtype, "out", 2)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2):
        raise KernelError("silu_mul: out must be [T, I] for gate_up [T, 2I]")
    _check(_fn("activation", "vl_silu_mul")(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I2 // 2, int(group),
                                            _stream()), "vl_silu_mul")
    return out


ACTIVATIONS = {"silu": 0, "relu": 1, "capped_swish": 2}
# functions of ONE argument (an expert without a gate: down(f(up h))); the codes continue the gated ones
UNARY_ACTIVATIONS = {"relu2": 16, "tanh": 17}           # the square of max(v, 0); tanh


def _act_code(act) -> int:
    """The kernels' code of an activation name (None: -1); codes from 16 on are functions of one argument."""
    if act is None:
        return -1
    return ACTIVATIONS[act] if act in ACTIVATIONS else UNARY_ACTIVATIONS[act]


def unary_act(x, out, act):
    """out = f(x) element by element (float32 inside); f from UNARY_ACTIVATIONS."""
    _need(x, None, "x"); _need(out, x.dtype, "out")
    if x.numel() != out.numel():
        raise KernelError("unary_act: sizes differ")
    _check(_fn("activation", "vl_unary_act")(_ptr(x), _ptr(out), dtype_code(x.dtype), x.numel(), UNARY_ACTIVATIONS[act],
                                             _stream()), "vl_unary_act")
    return out


def gated_act(gate_up, out, act, group=0, alpha=1.0, limit=0.0, shift=0.0, bias=None):
    """out[t, i] = f(gate_i, up_i) of gate_up [T, 2I] in the layouts of `silu_mul`.  act: "silu" (silu(g) u),
    "relu" (max(g, 0) u) or "capped_swish" (g' = min(g, limit), u' = clamp(u, -limit, limit):
    g' sigmoid(alpha g') (u' + shift); limit <= 0: none).  `bias` (float32 [2I]) is added to gate_up first."""
    _need(gate_up, None, "gate_up", 2); _need(out, gate_up.dtype, "out", 2)
    T, I2 = gate_up.shape
    if I2 % 2 or out.shape != (T, I2 // 2):
        raise KernelError("gated_act: out must be [T, I] for gate_up [T, 2I]")
    if act not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation {act!r}; known: {', '.join(ACTIVATIONS)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
        if bias.shape[0] != I2:
            raise KernelError("gated_act: the bias has one entry per column of gate_up")
    _check(_fn("activation", "vl_gated_act")(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I2 // 2, int(group),
                                             ACTIVATIONS[act], float(alpha), float(limit), float(shift), _ptr(bias), _stream()),
           "vl_gated_act")
    return out


def scaled_sum(a, scale_a, b, scale_b, out):
    """out = scale_a * a + scale_b * b, element by element in float32; all three in one dtype and shape."""
    _need(a, None, "a"); _need(b, a.dtype, "b"); _need(out, a.dtype, "out")
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError("scaled_sum: shapes differ")
    _check(_fn("activation", "vl_scaled_sum")(_ptr(a), float(scale_a), _ptr(b), float(scale_b), _ptr(out), dtype_code(a.dtype),
                                              a.numel(), _stream()), "vl_scaled_sum")
    return out


def scale_softcap(logits, scale, cap):
    """In place on float32 logits: z <- cap * tanh(z * scale / cap) (cap <= 0 or None: only the scale)."""
    _need(logits, torch.float32, "logits")
    _check(_fn("activation", "vl_scale_softcap")(_ptr(logits), logits.numel(), float(scale), float(cap or 0.0), _stream()),
           "vl_scale_softcap")
    return logits


# ---------------------------------------------------------------- layer norm
def layernorm_add(y, weight, eps, x, cast=None):
    """x[r] += layer_norm(y[r]) * weight (no bias; float32 arithmetic); x float32 [T, H], y in the activation
    dtype.  `cast` (activation dtype, [T, H]) receives the new x."""
    _need(y, None, "y", 2); _need(weight, torch.float32, "weight", 1); _need(x, torch.float32, "x", 2)
    if y.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError(f"layernorm_add: shapes disagree: y {tuple(y.shape)}, x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if cast is not None:
        _need(cast, y.dtype, "cast", 2)
        if cast.shape != x.shape:
            raise KernelError("layernorm_add: cast must have the stream's shape")
    _check(_fn("embed_norm", "vl_layernorm_add")(_ptr(y), dtype_code(y.dtype), _ptr(weight), float(eps), _ptr(x), _ptr(cast),
                                                 x.shape[0], x.shape[1], _stream()), "vl_layernorm_add")
    return x


def rmsnorm_add(y, weight, eps, mult, x, cast=None, bias=None, pair=None):
    """x[r] += mult * (y[r] / sqrt(mean(y[r]^2) + eps) * weight), x float32 [R, H], y in the activation dtype; `cast`
    (same dtype as y, or None) receives the new x.  `bias` (float32 [H] or None) is added to every row of y first.
    `pair` = (y2, s1, s2): the normed row is s1 * y + s2 * y2 (the results of two sub-layers side by side), in float32."""
    y2, s1, s2 = pair if pair is not None else (None, 1.0, 0.0)
    if y2 is not None:
        _need(y2, y.dtype, "y2", 2)
        if y2.shape != y.shape:
            raise KernelError("rmsnorm_add: the two rows of a pair have one shape")
    _need(y, None, "y", 2); _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1)
    if y.shape != x.shape or weight.shape[0] != x.shape[1]:
        raise KernelError(f"rmsnorm_add: y {tuple(y.shape)}, x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if cast is not None:
        _need(cast, y.dtype, "cast", 2)
        if cast.shape != x.shape:
            raise KernelError("rmsnorm_add: cast must have the shape of x")
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
        if bias.shape[0] != x.shape[1]:
            raise KernelError("rmsnorm_add: the bias has one entry per column")
    _check(_fn("embed_norm", "vl_rmsnorm_add")(_ptr(y), dtype_code(y.dtype), _ptr(bias), _ptr(weight), float(eps), float(mult), _ptr(x),
                                               _ptr(cast), x.shape[0], x.shape[1], _ptr(y2), float(s1), float(s2), _stream()),
           "vl_rmsnorm_add")
    return x


def layernorm_rows(x, rows, weight, eps, out):
    """out[r] = layer_norm(x[rows[r]]) * weight (rows None: every row); x float32."""
    _need(x, torch.float32, "x", 2); _need(weight, torch.float32, "weight", 1); _need(out, None, "out", 2)
    R = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    if out.shape != (R, x.shape[1]) or weight.shape[0] != x.shape[1]:
        raise KernelError("layernorm_rows: shapes disagree")
    _check(_fn("embed_norm", "vl_layernorm_rows")(_ptr(x), _ptr(rows), _ptr(weight), float(eps), _ptr(out),
                                                  dtype_code(out.dtype), R, x.shape[1], _stream()), "vl_layernorm_rows")
    return out


# ---------------------------------------------------------------- latent attention
def latent_norm_write(proj, q_rank, kv_rank, q_weight, kv_weight, eps, cq_out, slots, cache, err, rot_dim=0, rotary=None,
                      positions=None):
    """proj [T, >= q_rank + kv_rank] = [a_q | a_kv]: cq_out [T, q_rank] = rmsnorm(a_q) * q_weight; the cache row
    `slots[t]` of `cache` [pages, 1, page_size, width >= kv_rank] = rmsnorm(a_kv) * kv_weight, zero beyond kv_rank
    (slots None or negative: no write).  `rot_dim` > 0: proj carries rot_dim more columns behind a_kv, a key part that is
    not normed; `rotary` (inv_freq float32 [rot / 2], rot) turns its first rot features by `positions`, and the part is
    written into the cache row behind the latent."""
    inv_freq, rot = rotary if rotary is not None else (None, 0)
    if rot_dim:
        if rot:
            _need(inv_freq, torch.float32, "inv_freq", 1); _need(positions, torch.int32, "positions", 1)
            if inv_freq.shape[0] != rot // 2 or positions.shape[0] != proj.shape[0]:
                raise KernelError("latent_norm_write: inv_freq holds rot / 2 numbers, positions one per token")
        if proj.shape[1] < q_rank + kv_rank + rot_dim or (slots is not None and cache.shape[3] < kv_rank + rot_dim):
            raise KernelError("latent_norm_write: no room for the rotated key part")
    _need(proj, None, "proj", 2); _need(cq_out, proj.dtype, "cq_out", 2)
    _need(q_weight, torch.float32, "q_weight", 1); _need(kv_weight, torch.float32, "kv_weight", 1)
    T = proj.shape[0]
    if proj.shape[1] < q_rank + kv_rank or cq_out.shape != (T, q_rank) or q_weight.shape[0] != q_rank \
            or kv_weight.shape[0] != kv_rank:
        raise KernelError("latent_norm_write: shapes disagree")
    width, num_slots = kv_rank, 0
    if slots is not None:
        _need(slots, torch.int32, "slots", 1); _need(cache, proj.dtype, "cache", 4)
        if cache.shape[1] != 1 or cache.shape[3] < kv_rank or slots.shape[0] < T:
            raise KernelError(f"latent_norm_write: cache {tuple(cache.shape)} does not hold rows of {kv_rank}")
        width, num_slots = cache.shape[3], cache.shape[0] * cache.shape[2]
    _check(_fn("latent", "vl_latent_norm_write")(
        _ptr(proj), dtype_code(proj.dtype), proj.shape[1], T, int(q_rank), int(kv_rank), _ptr(q_weight), _ptr(kv_weight),
        float(eps), _ptr(cq_out), _ptr(slots), _ptr(cache) if slots is not None else None, max(width, kv_rank + rot_dim),
        num_slots, int(rot_dim), int(rot if rot_dim else 0), _ptr(inv_freq) if rot_dim else None,
        _ptr(positions) if rot_dim and rot else None, _ptr(err), _stream()), "vl_latent_norm_write")
    return cq_out


def rope_heads(x, col0, stride, heads, inv_freq, rot, positions):
    """In place on x [T, ld]: the features col0 + h * stride + [0, rot) of every head h < heads are turned by the token's
    position (pairs (i, i + rot/2), angle = position * inv_freq[i] in float32)."""
    _need(x, None, "x", 2); _need(inv_freq, torch.float32, "inv_freq", 1); _need(positions, torch.int32, "positions", 1)
    if inv_freq.shape[0] != rot // 2 or positions.shape[0] != x.shape[0]:
        raise KernelError("rope_heads: inv_freq holds rot / 2 numbers, positions one per token")
    _check(_fn("latent", "vl_rope_heads")(_ptr(x), dtype_code(x.dtype), x.shape[0], x.shape[1], int(col0), int(stride), int(heads),
                                          int(rot), _ptr(inv_freq), _ptr(positions), _stream()), "vl_rope_heads")
    return x


def head_norm_write(qkv, positions, slots, q_weight, k_weight, eps, qk_dim, v_norm, v_dim, q_temp, k_cache, v_cache,
                    num_heads, num_kv_heads, head_dim, err, v_eps=None):
    """The head work of an attention without rotation, in place on the q part of qkv [T, >= (nq + 2 nkv) hd] and into the
    cache slots: q and k heads divided by their root mean square over their first `qk_dim` features (0: no norm; weights
    float32 [hd] or None), the query times 1 + coef ln(floor((pos + 1) / every) + 1) for `q_temp` = (coef, every), every
    value head divided by its root mean square over `v_dim` features when `v_norm`."""
    _need(qkv, None, "qkv", 2); _need(positions, torch.int32, "positions", 1)
    T = qkv.shape[0]
    for w, n in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, torch.float32, n, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"head_norm_write: {n} has one entry per feature of a head")
    num_slots, page_size = 0, 1
    if slots is not None:
        _need(slots, torch.int32, "slots", 1); _need(k_cache, qkv.dtype, "k_cache", 4); _need(v_cache, qkv.dtype, "v_cache", 4)
        if k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or slots.shape[0] < T:
            raise KernelError(f"head_norm_write: cache {tuple(k_cache.shape)} does not match {num_kv_heads} heads of {head_dim}")
        num_slots, page_size = k_cache.shape[0] * k_cache.shape[2], k_cache.shape[2]
    coef, every = q_temp if q_temp is not None else (0.0, 0)
    _check(_fn("rope_cache", "vl_head_norm_write")(
        _ptr(qkv), dtype_code(qkv.dtype), _ptr(positions), _ptr(slots), _ptr(q_weight), _ptr(k_weight), float(eps), int(qk_dim),
        int(bool(v_norm)), int(v_dim), float(eps if v_eps is None else v_eps), float(coef), int(every),
        _ptr(k_cache) if slots is not None else None,
        _ptr(v_cache) if slots is not None else None, T, num_heads, num_kv_heads, head_dim, page_size, num_slots, qkv.shape[1],
        _ptr(err), _stream()), "vl_head_norm_write")
    return qkv


def sigmoid_gate(x, gate, gate_col=0):
    """In place: x[t, i] *= sigmoid(gate[t, gate_col + i]) for every column i of x [T, n] (float32 inside)."""
    _need(x, None, "x", 2); _need(gate, x.dtype, "gate", 2)
    T, n = x.shape
    if gate.shape[0] != T or gate_col + n > gate.shape[1]:
        raise KernelError("sigmoid_gate: the gate's columns leave its rows")
    _check(_fn("activation", "vl_sigmoid_gate")(_ptr(x), n, _ptr(gate), gate.shape[1], int(gate_col), dtype_code(x.dtype), T, n,
                                                _stream()), "vl_sigmoid_gate")
    return x


def gemm_heads(a, w, out):
    """One product per head on column slices: a [T, H*K], w [H, N, K], out [T, H*N];
    out[:, h*N:(h+1)*N] = a[:, h*K:(h+1)*K] @ w[h]^T.  float32 accumulation in a fixed order over K."""
    _need(a, None, "a", 2); _need(w, a.dtype, "w", 3); _need(out, a.dtype, "out", 2)
    H, N, K = w.shape
    T = a.shape[0]
    if a.shape[1] != H * K or out.shape != (T, H * N):
        raise KernelError(f"gemm_heads: shapes disagree a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("gemm_batched", "vl_gemm_batched_nt")(
        _ptr(a), _ptr(w), _ptr(out), dtype_code(a.dtype), T, N, K, H * K, K, H * N, K, N * K, N, H, None, 0,
        16 if T <= 16 else 64, _stream()), "vl_gemm_batched_nt")
    return out


def gemm_grouped(rows, w, out, tile_group, bm):
    """rows [cap, K] sorted by group in tiles of `bm` rows (`moe_align`), w [G, N, K], out [cap, N]:
    tile y is multiplied by w[tile_group[y]]; tiles with a negative group are skipped."""
    _need(rows, None, "rows", 2); _need(w, rows.dtype, "w", 3); _need(out, rows.dtype, "out", 2)
    _need(tile_group, torch.int32, "tile_group", 1)
    G, N, K = w.shape
    cap = rows.shape[0]
    if rows.shape[1] != K or out.shape != (cap, N) or cap % bm or tile_group.shape[0] < cap // bm:
        raise KernelError("gemm_grouped: shapes disagree")
    _check(_fn("gemm_batched", "vl_gemm_batched_nt")(
        _ptr(rows), _ptr(w), _ptr(out), dtype_code(rows.dtype), cap, N, K, K, K, N, 0, 0, 0, 1, _ptr(tile_group), N * K,
        int(bm), _stream()), "vl_gemm_batched_nt")
    return out


def gemm_grouped_fused_ok(dtype, K, N, act=None) -> bool:
    """Whether `gemm_grouped_fused` takes a product of these sizes (bfloat16, rows on 16-byte boundaries;
    with an activation, gate and up rows interleaved in blocks of 8, so N a multiple of 16)."""
    if dtype != torch.bfloat16:
        return False
    fn = build.load("gemm_batched").vl_gemm_grouped_fused_ok
    fn.argtypes, fn.restype = [c_int, c_int, c_int], c_int
    return bool(fn(int(K), int(N), _act_code(act)))


def gemm_grouped_fused(a, w, out, tile_group, bm, row_index, index_div, row_scale=None, act=None, alpha=1.0, limit=0.0,
                       shift=0.0):
    """The grouped product with a routed feed-forward's neighbours folded in (bfloat16, tensor cores):
    sorted row m is row row_index[m] // index_div of a [rows, K] (negative: zeros), times w[tile_group[y]]
    ([G, N, K]); the float32 sums are multiplied by row_scale[row_index[m]] when given; with `act`, w holds
    blocks of 8 gate rows and their 8 up rows and out is [cap, N / 2] = act(gate, up), else out is [cap, N]; an `act`
    of UNARY_ACTIVATIONS is applied to every column of a plain w (out [cap, N])."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 3); _need(out, torch.bfloat16, "out", 2)
    _need(tile_group, torch.int32, "tile_group", 1); _need(row_index, torch.int32, "row_index", 1)
    G, N, K = w.shape
    cap = row_index.shape[0]
    width = N // 2 if act in ACTIVATIONS else N
    if a.shape[1] != K or out.shape != (cap, width) or cap % bm or tile_group.shape[0] < cap // bm:
        raise KernelError("gemm_grouped_fused: shapes disagree")
    if row_scale is not None:
        _need(row_scale, torch.float32, "row_scale")
    _check(_fn("gemm_batched", "vl_gemm_grouped_fused")(
        _ptr(a), _ptr(w), _ptr(out), cap, N, K, K, width, _ptr(tile_group), N * K, int(bm), _ptr(row_index), int(index_div),
        _ptr(row_scale), _act_code(act), float(alpha), float(limit), float(shift), _stream()),
        "vl_gemm_grouped_fused")
    return out


# ---------------------------------------------------------------- routed experts
ROUTER_SCORES = {"sigmoid": 0, "softmax": 1}


def moe_sorted_rows(npairs, num_experts, bm) -> int:
    """Rows of the buffers that hold `npairs` (token, choice) pairs sorted by expert in tiles of bm rows."""
    need = npairs + min(num_experts, npairs) * (bm - 1)
    return -(-need // bm) * bm


def router_slices(K) -> int:
    """Parts into which the router's product cuts K (each a block's share; the parts' sums are added in order).
    A function of K alone, so that a token's logits do not depend on the step it is in."""
    for parts in (8, 4, 2):
        if K % (parts * 256) == 0:
            return parts
    return 1


def moe_route(h, router, top, ids, weights, logits, score="sigmoid", renormalize=False, groups=1, keep_groups=1, bias=None,
              choice_bias=None, group_top=1, renorm_eps=0.0):
    """h [T, K], router [E, K] (float32; or bfloat16 as stored, beside bfloat16 rows: products of two bfloat16 numbers
    are exact in float32, so the tensor cores' float32 sums are the 32-bit logits of the rounded rows):
    logits float32 [router_slices(K), T, E] = partial sums of h router^T; ids int32 [T, top] = the experts with
    the largest logits, weights float32 [T, top] = their scores (divided by their sum when `renormalize`).
    `groups` > 1: the experts form that many equal groups of neighbours, a group counts by its largest logit, and only
    experts of the `keep_groups` best groups are chosen from (scores are still taken over all experts).
    `bias` (float32 [E]) is added to the logits before anything else.  "softmax" with `renormalize` is the softmax
    over the chosen logits alone.  `choice_bias` (float32 [E]): experts and groups are chosen by score + choice_bias
    instead (the weights stay the scores without it); `group_top`: a group counts by the sum of that many of its largest
    choice values; `renorm_eps` is added to the sum that `renormalize` divides by."""
    _need(h, None, "h", 2); _need(router, None, "router", 2); _need(logits, torch.float32, "logits", 3)
    if router.dtype != torch.float32 and router.dtype != h.dtype:
        raise KernelError("moe_route: the router is float32, or bfloat16 beside bfloat16 rows")
    _need(ids, torch.int32, "ids", 2); _need(weights, torch.float32, "weights", 2)
    T, K = h.shape
    E = router.shape[0]
    slices = router_slices(K)
    if router.shape[1] != K or ids.shape != (T, top) or weights.shape != (T, top) or logits.shape != (slices, T, E):
        raise KernelError("moe_route: shapes disagree (logits: [router_slices(K), T, E])")
    _check(_fn("gemm_batched", "vl_gemm_rows_f32w")(_ptr(h), dtype_code(h.dtype), _ptr(router), dtype_code(router.dtype),
                                                    _ptr(logits), T, E, K, slices, _stream()), "vl_gemm_rows_f32w")
    if groups < 1 or E % groups or not 1 <= keep_groups <= groups or keep_groups * (E // groups) < top:
        raise KernelError(f"moe_route: {E} experts in {groups} groups, {keep_groups} kept, top {top}")
    if bias is not None:
        _need(bias, torch.float32, "bias", 1)
        if bias.shape[0] != E:
            raise KernelError(f"moe_route: the router's bias has {bias.shape[0]} entries for {E} experts")
    if choice_bias is not None:
        _need(choice_bias, torch.float32, "choice_bias", 1)
        if choice_bias.shape[0] != E:
            raise KernelError(f"moe_route: the choice bias has {choice_bias.shape[0]} entries for {E} experts")
    _check(_fn("moe", "vl_moe_route")(_ptr(logits), slices, T, E, int(top), ROUTER_SCORES[score], int(bool(renormalize)),
                                      int(groups), int(keep_groups), _ptr(bias), _ptr(choice_bias), int(group_top),
                                      float(renorm_eps), _ptr(ids), _ptr(weights), _stream()),
           "vl_moe_route")


TC5_GROUPED_TILE = 128    # rows per tile of the grouped tcgen05 product


def gemm_grouped_tc5_ok(dtype, pairs, num_experts, K) -> bool:
    """Whether a routed feed-forward of `pairs` (token, choice) rows runs its products on the tcgen05 tensor cores:
    bfloat16, rows on 16-byte boundaries, and enough rows that the experts' tiles of 128 rows are mostly full."""
    return dtype == torch.bfloat16 and K % 8 == 0 and pairs >= max(1024, 96 * num_experts)


def gemm_grouped_tc5(rows, w, out, tile_group, err, row_index=None, row_scale=None, act=None, alpha=1.0, limit=0.0, shift=0.0):
    """The grouped product on the tcgen05 tensor cores: rows [cap, K] sorted in tiles of 128, w [G, N, K], out [cap, N]
    or, with `act` (w then interleaves 8 gate rows with their 8 up rows), [cap, N / 2] = act(gate, up).
    row_scale: the float32 sums of row m are multiplied by row_scale[row_index[m]] first."""
    _need(rows, torch.bfloat16, "rows", 2); _need(w, torch.bfloat16, "w", 3); _need(out, torch.bfloat16, "out", 2)
    _need(tile_group, torch.int32, "tile_group", 1)
    G, N, K = w.shape
    cap = rows.shape[0]
    if rows.shape[1] != K or out.shape != (cap, N // 2 if act in ACTIVATIONS else N) or cap % TC5_GROUPED_TILE \
            or tile_group.shape[0] < cap // TC5_GROUPED_TILE:
        raise KernelError("gemm_grouped_tc5: shapes disagree")
    _check(_fn("gemm_tc5_grouped", "vl_gemm_bf16_tc5_grouped")(
        _ptr(rows), _ptr(w), _ptr(out), cap, N, K, G, _ptr(tile_group), _ptr(row_index), _ptr(row_scale),
        _act_code(act), float(alpha), float(limit), float(shift), _ptr(err), _stream()),
        "vl_gemm_bf16_tc5_grouped")
    return out


def moe_align(ids, num_experts, bm, sorted_rows, tile_group, place):
    _need(ids, torch.int32, "ids"); _need(sorted_rows, torch.int32, "sorted_rows", 1)
    _need(tile_group, torch.int32, "tile_group", 1); _need(place, torch.int32, "place", 1)
    n, cap = ids.numel(), sorted_rows.shape[0]
    if cap != moe_sorted_rows(n, num_experts, bm) or tile_group.shape[0] < cap // bm or place.shape[0] < n:
        raise KernelError("moe_align: buffer sizes do not match the number of pairs")
    _check(_fn("moe", "vl_moe_align")(_ptr(ids), n, int(num_experts), int(bm), cap, _ptr(sorted_rows), _ptr(tile_group),
                                      _ptr(place), _stream()), "vl_moe_align")


def moe_gather(h, sorted_rows, weights, top, rows, scale_input):
    _need(h, None, "h", 2); _need(rows, h.dtype, "rows", 2); _need(weights, torch.float32, "weights")
    if rows.shape != (sorted_rows.shape[0], h.shape[1]):
        raise KernelError("moe_gather: shapes disagree")
    _check(_fn("moe", "vl_moe_gather")(_ptr(h), dtype_code(h.dtype), _ptr(sorted_rows), _ptr(weights), rows.shape[0],
                                       int(top), h.shape[1], int(bool(scale_input)), _ptr(rows), _stream()), "vl_moe_gather")
    return rows


def moe_combine(result, place, weights, top, out, scale_output, add=None):
    """out[t] = the sum over token t's choices (in their order) of (weight *) result[place[t, j]]; `add` [T, N]: one more
    row per token, added last (a feed-forward that every token passes)."""
    _need(result, None, "result", 2); _need(out, result.dtype, "out", 2); _need(weights, torch.float32, "weights")
    T, N = out.shape
    if result.shape[1] != N or place.shape[0] < T * top:
        raise KernelError("moe_combine: shapes disagree")
    if add is not None:
        _need(add, out.dtype, "add", 2)
        if add.shape != out.shape:
            raise KernelError("moe_combine: the added rows have the output's shape")
    _check(_fn("moe", "vl_moe_combine")(_ptr(result), dtype_code(result.dtype), _ptr(place), _ptr(weights), T, int(top), N,
                                        int(bool(scale_output)), _ptr(out), _ptr(add), _stream()), "vl_moe_combine")
    return out


# ---------------------------------------------------------------- matrix products
def gemm_f32(a, w, out):
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, fixed order over K)."""
    _need(a, torch.float32, "a", 2); _need(w, torch.float32, "w", 2); _need(out, torch.float32, "out", 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes disagree a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _check(_fn("gemm_f32", "vl_gemm_f32_nt")(_ptr(a), _ptr(w), _ptr(out), M, N, K, K, K, N, _stream()), "vl_gemm_f32_nt")
    return out


SMALL_M = 16              # most rows of the weight-streaming product, which is also what its kernel takes; measured at
                          # Qwen3-8B sizes, context 4,096: batch 12 decodes in 5.00 ms against 5.18 ms with the library
                          # product from 9 rows on, batch 16 in 5.42 against 5.60 (the norms and SwiGLU run inside it)


def gemm_bf16_small_m_ok(M, K) -> bool:
    return 0 < M <= SMALL_M and K % 8 == 0


def _gemm_shapes(a, w, out, swiglu):
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, None, "out", 2)
    M, K = a.shape
    N = w.shape[0]
    width = N // 2 if swiglu else N
    if w.shape[1] != K or out.shape != (M, width) or (swiglu and N % (2 * SWIGLU_GROUP)):
        raise KernelError(f"gemm_bf16: shapes disagree a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}"
                          + (" (fused SwiGLU)" if swiglu else ""))
    return M, N, K, width


NORM_PARTIALS = 1024      # vectors of 16 partial sums a product kernel may leave (at least its number of blocks)


def gemm_bf16_small_m(a, w, out, err=None, swiglu=False, scaled=None, sink=None):
    """out[M, N] = a[M, K] @ w[N, K]^T for M <= 16: bfloat16 operands, float32 accumulation,
    out bfloat16 or float32.  Bound by one read of w.  swiglu: w holds blocks of 8 gate rows and
    their 8 up rows, out is [M, N/2] = silu(gate) * up.
    scaled = (partial float32 [>= count, 16], count, eps, size): the rows of `a` are an RMS norm's
    output without its scales; row m of the result is scaled by 1/sqrt(sum_b partial[b, m]/size + eps).
    sink = (x float32 [M, N], next_weight float32 [N], partial_out float32 [NORM_PARTIALS, 16]): the
    result is added into x, out receives bf16(x * next_weight) and partial_out the sums of squares of x
    block by block; returns the number of vectors written instead of out."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    ss_in, count, eps, size = (None, 0, 0.0, 0) if scaled is None else scaled
    x, next_w, ss_out = (None, None, None) if sink is None else sink
    if scaled is not None:
        _need(ss_in, torch.float32, "partial", 2)
        if ss_in.shape[1] != 16 or not 0 < count <= ss_in.shape[0] or size != K:
            raise KernelError("gemm_bf16_small_m: partial sums do not match the product")
    grid = ctypes.c_int(0)
    if sink is not None:
        _need(x, torch.float32, "x", 2); _need(next_w, torch.float32, "next_weight", 1)
        _need(ss_out, torch.float32, "partial_out", 2)
        if x.shape != (M, N) or next_w.shape[0] != N or ss_out.shape != (NORM_PARTIALS, 16) or swiglu:
            raise KernelError("gemm_bf16_small_m: the stream, the next weight or the partial sums do not match")
    _check(_fn("gemm_bf16", "vl_gemm_bf16_small_m_fused")(
        _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, K, K, width, _ptr(err), int(swiglu),
        _ptr(ss_in), int(count), float(eps), int(size), _ptr(x), N, _ptr(next_w), _ptr(ss_out),
        ctypes.addressof(grid) if sink is not None else None, _stream()), "vl_gemm_bf16_small_m")
    if sink is not None:
        if not 0 < grid.value <= NORM_PARTIALS:
            raise KernelError(f"gemm_bf16_small_m: {grid.value} blocks do not fit the partial sums")
        return grid.value
    return out


# From this many rows on the tcgen05 kernels are used: 1,024 where the activation is fused into the product
# (the library would need a kernel of its own for it: level at 1,024 rows, ahead beyond), 2,048 for a plain
# product (measured at 1,024 rows, q/k/v and down of Qwen3-8B: 58 and 82 us against the library's 41 and 73;
# at 2,048 rows 81 and 156 against 72 and 137; at 4,096 rows 158 and 358 against 165 and 314).
TC5_MIN_M = 1024
TC5_MIN_M_PLAIN = 2048


def gemm_bf16_tc5_ok(M, K, fused=False) -> bool:
    return M >= (TC5_MIN_M if fused else TC5_MIN_M_PLAIN) and K % 8 == 0


def gemm_bf16_tc5(a, w, out, err=None, swiglu=False):
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA tiles, accumulators in
    TMEM): bfloat16 operands, float32 accumulation, out bfloat16 or float32.  For many rows.
    swiglu: as in `gemm_bf16_small_m`."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    _check(_fn("gemm_tc5", "vl_gemm_bf16_tc5")(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K,
                                               K, K, width, _ptr(err), int(swiglu), _stream()), "vl_gemm_bf16_tc5")
    return out


_sm_pairs = None


def sm_pairs() -> int:
    """Pairs of SMs of the current device (what a kernel of two-block clusters can keep busy)."""
    global _sm_pairs
    if _sm_pairs is None:
        _sm_pairs = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count // 2
    return _sm_pairs


def gemm_bf16_tc5_pair(a, w, out, err=None, swiglu=False):
    """As `gemm_bf16_tc5`, with two SMs on one 256 x 256 tile (tcgen05.mma.cta_group::2): each SM
    brings its rows of a and half of the tile's rows of w into shared memory."""
    M, N, K, width = _gemm_shapes(a, w, out, swiglu)
    _check(_fn("gemm_tc5_pair", "vl_gemm_bf16_tc5_pair")(_ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K,
                                                         K, K, width, _ptr(err), int(swiglu), _stream()),
           "vl_gemm_bf16_tc5_pair")
    return out


# ---------------------------------------------------------------- measurement
def read_only(buf, nbytes=None, sink=None):
    """Streams the first `nbytes` bytes of `buf` from memory once and does nothing with them: the time of
    this launch is what any kernel that must read as many bytes is measured against (bench.py --read-ceiling)."""
    _need(buf, None, "buf")
    total = buf.numel() * buf.element_size()
    nbytes = total if nbytes is None else int(nbytes)
    if not 0 < nbytes <= total or nbytes % 16:
        raise KernelError(f"read_only: {nbytes} bytes of a buffer of {total} (a multiple of 16 is wanted)")
    _check(_fn("memprobe", "vl_read_only")(_ptr(buf), nbytes, _ptr(sink), _stream()), "vl_read_only")


# ---------------------------------------------------------------- sampling
def apply_penalties(logits, seen_off=None, seen_ids=None, repeat=None, presence=None,
                    bias_off=None, bias_ids=None, bias_vals=None):
    _need(logits, torch.float32, "logits", 2)
    R, V = logits.shape
    _check(_fn("sampling", "vl_apply_penalties")(
        _ptr(logits), logits.stride(0), R, V, _ptr(seen_off), _ptr(seen_ids), _ptr(repeat), _ptr(presence),
        _ptr(bias_off), _ptr(bias_ids), _ptr(bias_vals), _stream()), "vl_apply_penalties")
    return logits


def sample(logits, temperature, top_k, top_p, uniform, out_token, out_logprob=None):
    _need(logits, torch.float32, "logits", 2); _need(out_token, torch.int32, "out_token", 1)
    R, V = logits.shape
    for t, dt, n in ((temperature, torch.float32, "temperature"), (top_k, torch.int32, "top_k"),
                     (top_p, torch.float32, "top_p"), (uniform, torch.float32, "uniform"),
                     (out_logprob, torch.float32, "out_logprob")):
        if t is not None:
            _need(t, dt, n, 1)
            if t.shape[0] < R:
                raise KernelError(f"{n} has fewer entries than rows")
    _check(_fn("sampling", "vl_sample")(
        _ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform),
        _ptr(out_token), _ptr(out_logprob), _stream()), "vl_sample")
    return out_token


# ---------------------------------------------------------------- several residual streams, tanh norm
HC_MAX_STREAMS = 16


def hc_step(streams, *, single=None, y=None, mix=None, out_w=None, in_w=None, norm=None, h=None, total=None):
    """One pass over the streams float32 [T, S, H] (csrc/hyper.cu): spread from `single` [T, H], write a sub-layer's
    result `y` [T, H] back (mix [S, S] indexed [from, to], out_w [S]), read the next sub-layer's input into `h` [T, H]
    (in_w [S]; norm = (alpha, weight, bias) of the tanh norm, or None for the plain sum) and the sum of the streams
    into `total` float32 [T, H]; every part optional."""
    _need(streams, torch.float32, "streams", 3)
    T, S, H = streams.shape
    for t, n in ((single, "single"), (total, "total")):
        if t is not None:
            _need(t, torch.float32, n, 2)
            if t.shape != (T, H):
                raise KernelError(f"hc_step: {n} must be [{T}, {H}]")
    dt = None
    for t, n in ((y, "y"), (h, "h")):
        if t is not None:
            _need(t, None, n, 2)
            if t.shape != (T, H) or (dt is not None and t.dtype != dt):
                raise KernelError(f"hc_step: {n} must be [{T}, {H}] in one dtype")
            dt = t.dtype
    for t, n, shape in ((mix, "mix", (S, S)), (out_w, "out_w", (S,)), (in_w, "in_w", (S,))):
        if t is not None:
            _need(t, torch.float32, n)
            if tuple(t.shape) != shape:
                raise KernelError(f"hc_step: {n} must be {shape}")
    if (y is None) != (mix is None) or (y is None) != (out_w is None) or (in_w is None) != (h is None):
        raise KernelError("hc_step: y comes with mix and out_w, in_w with h")
    alpha = w = b = None
    if norm is not None:
        alpha, w, b = norm
        _need(alpha, torch.float32, "alpha"); _need(w, torch.float32, "weight", 1); _need(b, torch.float32, "bias", 1)
        if alpha.numel() != 1 or w.shape[0] != H or b.shape[0] != H:
            raise KernelError("hc_step: the norm's alpha is one number, its weight and bias have H entries")
    _check(_fn("hyper", "vl_hc_step")(_ptr(streams), _ptr(single), _ptr(y), dtype_code(dt or torch.float32), _ptr(mix),
                                      _ptr(out_w), _ptr(in_w), _ptr(alpha), _ptr(w), _ptr(b), _ptr(h), _ptr(total),
                                      T, S, H, _stream()), "vl_hc_step")


def dyt_rows(x, delta, rows, alpha, weight, bias, out):
    """out[r] = tanh(alpha * x[row r]) * weight + bias; x float32 [T, H] (+= delta first; stored when rows is None)."""
    _need(x, torch.float32, "x", 2); _need(out, None, "out", 2)
    _need(alpha, torch.float32, "alpha"); _need(weight, torch.float32, "weight", 1); _need(bias, torch.float32, "bias", 1)
    H = x.shape[1]
    R = x.shape[0] if rows is None else rows.shape[0]
    if alpha.numel() != 1 or weight.shape[0] != H or bias.shape[0] != H or out.shape != (R, H):
        raise KernelError("dyt_rows: shapes disagree")
    if delta is not None:
        _need(delta, out.dtype, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError("dyt_rows: delta must match x")
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
    _check(_fn("hyper", "vl_dyt_rows")(_ptr(x), _ptr(delta), _ptr(rows), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out),
                                       dtype_code(out.dtype), R, H, _stream()), "vl_dyt_rows")
    return out


# ---------------------------------------------------------------- recurrent mixers (csrc/recurrent.cu)
def scan_shape(n: int, columns: int):
    """(rows a lane, lanes a column, threads a block, columns a block, blocks a head) of a scan over a state of n rows and
    `columns` columns per head; the same arithmetic as csrc/recurrent.cu (scan_shape), on which the state's size rests."""
    if not 0 < n <= 512 or columns <= 0:
        raise KernelError(f"the scan kernels take states of 1 to 512 rows, got {n} x {columns}")
    rows = 4 if n <= 128 else (8 if n <= 256 else 16)
    L = 1
    while L * rows < n:
        L *= 2
    threads = 128 if 128 // L >= columns else (256 if 256 // L >= columns else 512)
    ct = threads // L
    return rows, L, threads, ct, -(-columns // ct)


def scan_lanes(n: int) -> int:
    return scan_shape(n, 1)[1]


def scan_state_floats(H, n, P) -> int:
    """Floats of a recurrence's state (H heads of n x P numbers) in the layout the scan kernels keep it in: per head
    and tile of columns, the rows each lane holds, thread by thread."""
    rows, _, threads, _, Z = scan_shape(n, P)
    return H * Z * rows * threads


def mlstm_state_floats(H, D, P) -> int:
    """The matrix memory's state: S as `scan_state_floats`, then a normaliser [D] and a running maximum for every tile
    of columns of every head."""
    Z = scan_shape(D, P)[4]
    return scan_state_floats(H, D, P) + H * Z * D + H * Z


def _state_args(state, state_off, need):
    _need(state, torch.float32, "state", 2)
    if state_off < 0 or state_off + need > state.shape[1]:
        raise KernelError(f"a state row of {state.shape[1]} floats cannot hold {need} at {state_off}")
    return state.data_ptr() + 4 * state_off, state.shape[1]


def _seg_args(cu, slots):
    _need(cu, torch.int32, "cu_seqlens", 1); _need(slots, torch.int32, "state_slots", 1)
    B = cu.shape[0] - 1
    if slots.shape[0] < B:
        raise KernelError("one state slot per request")
    return B


def short_conv(x, col0, C, weight, bias, state, state_off, cu, slots, out, act=True, longest=None, in_bias=None):
    """out float32 [T, C] = act(causal convolution over time of columns col0 .. col0+C of x [T, ld]); weight float32
    [C, taps]; the last taps-1 inputs live at `state_off` of every request's state row [(taps-1), C].  `longest`: a
    bound on the tokens one request brings (default: all of them).  `in_bias` (float32 [C] or None) is added to the
    rows of x as they are read, before the convolution; the state keeps them with it."""
    _need(x, None, "x", 2); _need(weight, torch.float32, "weight", 2)
    taps = weight.shape[1]
    if out is not None:                         # None: only the new state is made (the rows were computed elsewhere)
        _need(out, torch.float32, "out", 2)
    if weight.shape[0] != C or (out is not None and out.shape != (x.shape[0], C)):
        raise KernelError("short_conv: shapes disagree")
    for t, n in ((bias, "bias"), (in_bias, "in_bias")):
        if t is not None:
            _need(t, torch.float32, n, 1)
            if t.shape[0] != C:
                raise KernelError(f"short_conv: {n} has one entry per channel")
    B = _seg_args(cu, slots)
    sp, stride = _state_args(state, state_off, (taps - 1) * C)
    _check(_fn("recurrent", "vl_short_conv")(_ptr(x), dtype_code(x.dtype), x.shape[1], col0, C, _ptr(weight), _ptr(bias),
                                             _ptr(in_bias), taps,
                                             sp, stride, _ptr(cu), _ptr(slots), B, int(longest or max(x.shape[0], 1)), _ptr(out),
                                             int(bool(act)), _stream()), "vl_short_conv")
    if out is not None and int(longest or x.shape[0]) > 64:
        global launch_count
        launch_count += 1           # requests cut among blocks: the new state is a launch of its own
    return out


def ssd_scan(xbc, proj, dt_col, dt_bias, A_log, D, state, state_off, cu, slots, y, H, G, N, P):
    _need(xbc, torch.float32, "xbc", 2); _need(proj, None, "proj", 2); _need(y, torch.float32, "y", 2)
    for t, n in ((dt_bias, "dt_bias"), (A_log, "A_log"), (D, "D")):
        _need(t, torch.float32, n, 1)
        if t.shape[0] != H:
            raise KernelError(f"ssd_scan: {n} has one entry per head")
    T = xbc.shape[0]
    if proj.shape[0] != T or y.shape != (T, H * P) or dt_col + H > proj.shape[1]:
        raise KernelError("ssd_scan: shapes disagree")
    B = _seg_args(cu, slots)
    sp, stride = _state_args(state, state_off, scan_state_floats(H, N, P))
    _check(_fn("recurrent", "vl_ssd_scan")(_ptr(xbc), xbc.shape[1], _ptr(proj), dtype_code(proj.dtype), proj.shape[1], dt_col,
                                           _ptr(dt_bias), _ptr(A_log), _ptr(D), sp, stride, _ptr(cu), _ptr(slots), B, _ptr(y),
                                           H, G, N, P, _stream()), "vl_ssd_scan")
    return y


def mlstm_scan(proj, q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, cap, q_scale, denom_eps, state, state_off, cu, slots, o, H, D, P):
    _need(proj, None, "proj", 2); _need(o, torch.float32, "o", 2)
    _need(i_bias, torch.float32, "i_bias", 1); _need(f_bias, torch.float32, "f_bias", 1)
    T, ld = proj.shape
    if o.shape != (T, H * P) or i_bias.shape[0] != H or f_bias.shape[0] != H:
        raise KernelError("mlstm_scan: shapes disagree")
    if max(q_col + H * D, k_col + H * D, v_col + H * P, i_col + H, f_col + H) > ld:
        raise KernelError("mlstm_scan: a column range leaves the rows")
    B = _seg_args(cu, slots)
    sp, stride = _state_args(state, state_off, mlstm_state_floats(H, D, P))
    _check(_fn("recurrent", "vl_mlstm_scan")(_ptr(proj), dtype_code(proj.dtype), ld, q_col, k_col, v_col, i_col, f_col,
                                             _ptr(i_bias), _ptr(f_bias), float(cap), float(q_scale), float(denom_eps), sp, stride, _ptr(cu),
                                             _ptr(slots), B, _ptr(o), H, D, P, _stream()), "vl_mlstm_scan")
    return o


def delta_scan(qkv, decay, decay_col, dt_bias, A_log, proj, beta_col, q_scale, unit_eps, state, state_off, cu, slots, o, H, G, D, P):
    _need(qkv, torch.float32, "qkv", 2); _need(decay, None, "decay", 2); _need(proj, decay.dtype, "proj", 2)
    _need(o, torch.float32, "o", 2); _need(dt_bias, torch.float32, "dt_bias", 1); _need(A_log, torch.float32, "A_log", 1)
    T = qkv.shape[0]
    if decay.shape[0] != T or decay_col + H * D > decay.shape[1] or proj.shape[0] != T or o.shape != (T, H * P) or dt_bias.shape[0] != H * D \
            or A_log.shape[0] != H or beta_col + H > proj.shape[1]:
        raise KernelError("delta_scan: shapes disagree")
    B = _seg_args(cu, slots)
    sp, stride = _state_args(state, state_off, scan_state_floats(H, D, P))
    _check(_fn("recurrent", "vl_delta_scan")(_ptr(qkv), qkv.shape[1], _ptr(decay), decay.shape[1], decay_col, _ptr(dt_bias), _ptr(A_log), _ptr(proj),
                                             dtype_code(proj.dtype), proj.shape[1], beta_col, float(q_scale), float(unit_eps),
                                             sp, stride, _ptr(cu), _ptr(slots), B, _ptr(o), H, G, D, P, _stream()),
           "vl_delta_scan")
    return o


def token_shift_multi(h, mu, state, state_off, cu, slots, req_index, positions, out):
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]: S mixes at once, h [T, W] and out [S, T, W] in one dtype, mu float32
    [S, W]; the row before a portion's first token is state[slot, state_off : state_off + W] (float32), which the launch
    replaces by the portion's last row."""
    _need(h, None, "h", 2); _need(mu, torch.float32, "mu", 2); _need(out, h.dtype, "out", 3)
    T, W = h.shape
    S = mu.shape[0]
    if mu.shape[1] != W or out.shape != (S, T, W) or req_index.shape[0] != T or positions.shape[0] != T:
        raise KernelError("token_shift_multi: shapes disagree")
    base, stride = _state_args(state, state_off, W)
    _seg_args(cu, slots)
    _need(req_index, torch.int32, "req_index", 1); _need(positions, torch.int32, "positions", 1)
    _check(_fn("recurrent", "vl_token_shift_multi")(_ptr(h), _ptr(mu), S, base, stride, _ptr(cu), _ptr(slots), _ptr(req_index),
                                                    _ptr(positions), _ptr(out), dtype_code(h.dtype), T, W, _stream()),
           "vl_token_shift_multi")
    return out


DECAY_SCAN_THREADS = 128


def decay_scan_shape(D: int, P: int):
    """(rows a lane, lanes a column, columns a block, blocks a head) of `decay_scan` over a state of D rows and P columns per
    head; the same arithmetic as csrc/recurrent.cu (decay_shape), on which the state's size rests."""
    if not 0 < D <= 512 or P <= 0:
        raise KernelError(f"decay_scan takes states of 1 to 512 rows, got {D} x {P}")
    rows = 4 if D <= 128 else (8 if D <= 256 else 16)
    L = 1
    while L * rows < D:
        L *= 2
    ct = DECAY_SCAN_THREADS // L
    return rows, L, ct, -(-P // ct)


def decay_state_floats(H, D, P) -> int:
    """Floats of `decay_scan`'s state (H heads of D x P numbers) in the layout the kernel keeps it in."""
    rows, _, _, Z = decay_scan_shape(D, P)
    return H * Z * rows * DECAY_SCAN_THREADS


def decay_from_raw(z, col, w0):
    """In place on columns col .. col + len(w0) of z [T, ld]: z <- exp(-exp(z + w0)), a decay in (0, 1) per column (float32 inside)."""
    _need(z, None, "z", 2); _need(w0, torch.float32, "w0", 1)
    if col < 0 or col + w0.shape[0] > z.shape[1]:
        raise KernelError("decay_from_raw: the columns leave the rows")
    _check(_fn("recurrent", "vl_decay_from_raw")(_ptr(z), dtype_code(z.dtype), z.shape[0], z.shape[1], int(col), _ptr(w0),
                                                 w0.shape[0], _stream()), "vl_decay_from_raw")
    return z


def decay_scan(r, k, v, w, u, state, state_off, cu, slots, o, H, D, P):
    """Per head a memory S [D, P] with a decay per key channel: o_t = (S + diag(u) k_t v_t^T)^T r_t, then
    S <- diag(w_t) S + k_t v_t^T.  r, k, w: (tensor [T, ld], first column) with H*D columns, v likewise with H*P, all of
    one dtype; u float32 [H*D] (the bonus of the current token); o float32 [T, H*P]; the state as `decay_state_floats(H, D, P)`."""
    (rt, rc), (kt, kc), (vt, vc), (wt, wc) = r, k, v, w
    for t, n in ((rt, "r"), (kt, "k"), (vt, "v"), (wt, "w")):
        _need(t, rt.dtype, n, 2)
    _need(o, torch.float32, "o", 2); _need(u, torch.float32, "u", 1)
    T = rt.shape[0]
    if kt.shape[0] != T or vt.shape[0] != T or wt.shape[0] != T or o.shape != (T, H * P) or u.shape[0] != H * D:
        raise KernelError("decay_scan: shapes disagree")
    B = _seg_args(cu, slots)
    sp, stride = _state_args(state, state_off, decay_state_floats(H, D, P))
    _check(_fn("recurrent", "vl_decay_scan")(_ptr(rt), rt.shape[1], int(rc), _ptr(kt), kt.shape[1], int(kc), _ptr(vt), vt.shape[1],
                                             int(vc), _ptr(wt), wt.shape[1], int(wc), dtype_code(rt.dtype), _ptr(u), sp,
                                             stride, _ptr(cu), _ptr(slots), B, _ptr(o), H, D, P, _stream()), "vl_decay_scan")
    return o


GATES = {None: 0, "silu": 1, "sigmoid": 2}


def gate_norm(y, gate, gate_col, gate_kind, gate_first, weight, eps, out, part):
    """out [T, W] = RMS norm of y float32 [T, W] over parts of `part` columns, times weight (W entries, or `part`
    entries shared by the parts), with a gate taken from columns gate_col .. of `gate`: out = rms(y * g) * w when
    gate_first, else rms(y) * w * g; g = silu or sigmoid of the gate's value."""
    _need(y, torch.float32, "y", 2); _need(out, None, "out", 2); _need(weight, torch.float32, "weight", 1)
    T, W = y.shape
    if out.shape != (T, W) or weight.shape[0] not in (W, part):
        raise KernelError("gate_norm: shapes disagree")
    ld = 0
    if gate is not None:
        _need(gate, out.dtype, "gate", 2)
        ld = gate.shape[1]
        if gate.shape[0] != T or gate_col + W > ld:
            raise KernelError("gate_norm: the gate's columns leave its rows")
    _check(_fn("recurrent", "vl_gate_norm")(_ptr(y), _ptr(gate), dtype_code(out.dtype), ld, gate_col, GATES[gate_kind if gate is not None else None],
                                            int(bool(gate_first)), _ptr(weight), weight.shape[0], float(eps), _ptr(out), T, W,
                                            part, _stream()), "vl_gate_norm")
    return out
