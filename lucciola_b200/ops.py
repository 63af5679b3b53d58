"""Tensor-level wrappers of the kernel library.

Each function checks what the kernel cannot check for itself (device, type,
contiguity), passes raw pointers and the stream to the C interface, and raises
`KernelError` with the library's message when a call is refused.  There is no
other implementation behind these functions: without the library they raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from .csrc import KernelLibraryError, library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dt}")


_SIGNATURES = {
    "lb_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_float, c_void_p,
                     c_void_p],
    "lb_layernorm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "lb_layernorm_add": [c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_void_p, c_float, c_float, c_void_p, c_int,
                         c_int, c_int, c_void_p],
    "lb_round_copy": [c_void_p, c_int, c_void_p, c_longlong, c_void_p],
    "lb_decay_recurrence": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_int, c_void_p],
    "lb_rmsnorm_gated": [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_float, c_float, c_int, c_int,
                         c_int, c_longlong, c_void_p],
    "lb_head_gate": [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_longlong, c_float, c_int, c_int, c_int, c_void_p],
    "lb_route_topk": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "lb_expert_dispatch": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "lb_expert_gemm": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong,
                       c_longlong, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "lb_expert_dispatch_padded": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "lb_expert_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lb_gemm_tcgen05_grouped": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_float,
                                c_void_p, c_int, c_void_p],
    "lb_expert_combine": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "lb_add_group_rmsnorm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_float, c_void_p],
    "lb_scale": [c_void_p, c_longlong, c_float, c_void_p],
    "lb_add_into": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "lb_causal_taps": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lb_causal_taps_state": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lb_latent_norm": [c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "lb_gated_recurrence": [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "lb_gemm_heads_mma": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                          c_longlong, c_longlong, c_void_p, c_longlong, c_void_p],
    "lb_gemm_plain_batched": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
                              c_longlong, c_longlong, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p],
    "lb_add_rmsnorm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "lb_rope_kv": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_float, c_void_p],
    "lb_rotate_rows": [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_float, c_int, c_int,
                       c_float, c_void_p],
    "lb_round_cols": [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p],
    "lb_attention_plain": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_float, c_void_p, c_int,
                           c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "lb_short_conv": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_int, c_int, c_int, c_int, c_void_p],
    "lb_short_conv_state": [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lb_state_recurrence": [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                            c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p],
    "lb_channel_decay": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "lb_gated_group_norm": [c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_longlong, c_void_p],
    "lb_bias_rmsnorm_cols": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p],
    "lb_pool_kv": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "lb_add_rmsnorm_pair": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                            c_float, c_void_p],
    "lb_rmsnorm_mix2": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_float, c_void_p],
    "lb_activation": [c_int, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_float, c_void_p],
    "lb_swiglu": [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_void_p],
    "lb_gemm_plain": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                      c_longlong, c_void_p],
    "lb_gemm_tcgen05": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_void_p,
                        c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p],
    "lb_gemm_tcgen05_addnorm": [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_void_p],
    "lb_upload": [c_void_p, c_void_p, c_longlong, c_void_p],
    "lb_zero_rows": [c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p],
    "lb_gemm_tcgen05_heads": [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p],
    "lb_attention_flash": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p],
    "lb_attention_flash_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p,
                              c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "lb_attention_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_longlong, c_void_p, c_void_p],
    "lb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
}

_fn_cache: dict[str, object] = {}


def _fn(name: str):
    f = _fn_cache.get(name)
    if f is None:
        lib = library()
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"the kernel library lacks {name}") from e
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn_cache[name] = f
    return f


def _call(name: str, *args) -> None:
    rc = _fn(name)(*args)
    if rc != 0:
        raise KernelError(library().lb_last_error().decode())


def hash_uniform(key: int, counter: int, i: int) -> float:
    """The sampler's uniform number for (request key, generated index, vocabulary index), on the host."""
    lib = library()
    f = lib.lb_hash_uniform
    f.argtypes = [c_ulonglong, c_uint, c_uint]
    f.restype = c_float
    return float(f(key, counter, i))


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, what: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the GPU")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, is {t.dtype}")


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def embedding(out: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, stream: int,
              pos_table: torch.Tensor | None = None, positions: torch.Tensor | None = None,
              sin_freq: torch.Tensor | None = None, scale: float = 1.0, copy: torch.Tensor | None = None) -> None:
    """out[t, :] = table[ids[t], :] * scale as float32; with a table of position vectors, + pos_table[positions[t], :]; with
    `sin_freq` (float64 [ceil(H / 2)]) instead + the sinusoidal vector whose entries 2i, 2i + 1 are the sine and
    cosine of positions[t] * sin_freq[i].  `copy` (float32, out's shape) receives the same rows a second time."""
    if copy is not None:
        _check(copy, "embedding copy", torch.float32)
        if copy.shape != out.shape:
            raise KernelError("the embedding's second copy has the first one's shape")
    _check(out, "embedding output", torch.float32); _check(ids, "token ids", torch.int32); _check(table, "embedding table")
    T, H = out.shape
    if sin_freq is not None:
        _check(sin_freq, "frequencies", torch.float64); _check(positions, "positions", torch.int32)
        if sin_freq.shape[0] != (H + 1) // 2:
            raise KernelError(f"{sin_freq.shape[0]} frequencies for rows of {H}")
    if pos_table is not None:
        _check(pos_table, "position table", table.dtype); _check(positions, "positions", torch.int32)
        if pos_table.shape[1] != H:
            raise KernelError(f"position vectors have {pos_table.shape[1]} values, the embedding {H}")
    _call("lb_embedding", out.data_ptr(), ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), T, H,
          table.shape[0], _ptr(pos_table), _ptr(positions), pos_table.shape[0] if pos_table is not None else 0, _ptr(sin_freq),
          float(scale), _ptr(copy), stream)


def add_group_rmsnorm(out: torch.Tensor, residual: torch.Tensor, deltas: tuple, weight: torch.Tensor, groups: int,
                      eps: float, stream: int, rows: torch.Tensor | None = None) -> None:
    """residual += sum of up to two deltas (when rows is None); out = the row's `groups` equal consecutive parts each
    divided by its own sqrt(mean(part^2) + eps), times weight; on `rows` if given."""
    _check(out, "norm output"); _check(residual, "residual", torch.float32); _check(weight, "norm weight", torch.float32)
    deltas = tuple(d for d in deltas if d is not None)
    if len(deltas) > 2:
        raise KernelError("the group norm adds at most two deltas")
    for d in deltas:
        _check(d, "delta", deltas[0].dtype)
        if d.shape != residual.shape:
            raise KernelError("a delta must have the residual's shape")
    if rows is not None:
        _check(rows, "row index", torch.int32)
    H = out.shape[-1]
    _call("lb_add_group_rmsnorm", out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(),
          _ptr(deltas[0]) if deltas else None, _ptr(deltas[1]) if len(deltas) > 1 else None,
          dtype_code(deltas[0].dtype) if deltas else F32, weight.data_ptr(), _ptr(rows), out.shape[0], H, groups, eps, stream)


def add_into(residual: torch.Tensor, delta: torch.Tensor, stream: int) -> None:
    """residual += delta, in place, the sum in float32."""
    _check(residual, "residual", torch.float32); _check(delta, "delta")
    if residual.shape != delta.shape:
        raise KernelError("residual and delta must have one shape")
    _call("lb_add_into", residual.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype), residual.numel(), stream)


def scale_(x: torch.Tensor, factor: float, stream: int) -> None:
    """x *= factor, in place, float32."""
    _check(x, "tensor to scale", torch.float32)
    _call("lb_scale", x.data_ptr(), x.numel(), factor, stream)


def causal_taps(out: torch.Tensor, h: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, step, stream: int) -> None:
    """out_t = h_t + sum_j weight[j, :] * h_(t - taps + 1 + j) over each sequence's tokens in order (weight [taps, width],
    oldest tap first); what lies before a portion is read from state[slot] ([taps - 1, width], oldest first).  The
    state is not changed."""
    _check(out, "convolution output", h.dtype); _check(h, "convolution input"); _check(weight, "taps", torch.float32)
    T, W = h.shape
    taps = weight.shape[0]
    if weight.shape[1] != W:
        raise KernelError(f"the taps are [{weight.shape[0]}, {weight.shape[1]}] for rows of {W}")
    if state is not None:
        _check(state, "convolution state", h.dtype)
    _call("lb_causal_taps", dtype_code(h.dtype), out.data_ptr(), h.data_ptr(), weight.data_ptr(), _ptr(state),
          step.token_seq.data_ptr(), step.cu_tokens.data_ptr(), step.state_slots.data_ptr(), T, W, taps, stream)


def causal_taps_state(state: torch.Tensor, h: torch.Tensor, taps: int, step, stream: int) -> None:
    """state[slot] = the last taps - 1 rows of (state[slot] ++ this step's rows of the sequence)."""
    _check(state, "convolution state", h.dtype); _check(h, "convolution input")
    _call("lb_causal_taps_state", dtype_code(h.dtype), state.data_ptr(), h.data_ptr(), step.cu_tokens.data_ptr(),
          step.state_slots.data_ptr(), step.num_seqs, h.shape[1], taps, stream)


def latent_norm(pre: torch.Tensor, q_col: int, kv_col: int, q_rank: int, kv_rank: int, q_w: torch.Tensor, kv_w: torch.Tensor,
                q_out: torch.Tensor, pages: torch.Tensor, step, block_table: torch.Tensor, page_size: int, eps: float,
                stream: int) -> None:
    """RMSNorm of the two latents in the float32 rows of `pre`: the query latent goes to q_out [T, q_rank], the
    key/value latent to the token's place in `pages` ([pages, 1, page_size, kv_rank])."""
    _check(pre, "down-projections", torch.float32); _check(q_w, "query latent norm", torch.float32)
    _check(kv_w, "latent norm", torch.float32); _check(q_out, "query latent"); _check(pages, "latent pages", q_out.dtype)
    _check(block_table, "block table", torch.int32)
    _call("lb_latent_norm", dtype_code(q_out.dtype), pre.data_ptr(), pre.stride(0), q_col, kv_col, q_rank, kv_rank,
          q_w.data_ptr(), kv_w.data_ptr(), q_out.data_ptr(), pages.data_ptr(), step.positions.data_ptr(),
          step.token_seq.data_ptr(), block_table.data_ptr(), pre.shape[0], page_size, block_table.shape[1], eps, stream)


def gated_recurrence(pre: torch.Tensor, q_col: int, f_col: int, v_col: int, bias: torch.Tensor, lower: torch.Tensor,
                     state: torch.Tensor, out: torch.Tensor, step, heads: int, dim: int, vdim: int, stream: int,
                     max_tokens_a_seq: int = 0) -> None:
    """The HGRN2 recurrence over this step's tokens: per head S <- diag(f) S + (1 - f) v^T, out = S^T q with
    q = silu(pre[:, q_col..]), f = lower + (1 - lower) sigmoid(pre[:, f_col..] + bias), v = pre[:, v_col..];
    state [slots + 1, heads, dim, vdim] float32 is read and written at each sequence's slot; out [T, heads * vdim] float32.
    `max_tokens_a_seq`: the most tokens any sequence brings, if the host knows it (0: unknown); steps of a few tokens a
    sequence run in a kernel made for them, with the same sums in the same order."""
    _check(pre, "input projections", torch.float32); _check(bias, "gate bias", torch.float32)
    _check(lower, "lower bound", torch.float32); _check(state, "recurrent state", torch.float32)
    _check(out, "recurrence output", torch.float32)
    _call("lb_gated_recurrence", pre.data_ptr(), pre.stride(0), q_col, f_col, v_col, bias.data_ptr(), lower.data_ptr(),
          state.data_ptr(), out.data_ptr(), step.cu_tokens.data_ptr(), step.state_slots.data_ptr(), step.num_seqs,
          heads, dim, vdim, max_tokens_a_seq, stream)


def gemm_heads(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int, gate: torch.Tensor | None = None) -> None:
    """y[t, h, :] = x[t, h, :] . w[h]^T for w [heads, N, K], one product a head, 32-bit sums: bfloat16 operands with K
    a multiple of 8 on the tensor cores, everything else on the ordinary pipes.
    With `gate` (float32 [T, >= heads * N], row-strided): y[t, h, n] *= sigmoid(gate[t, h * N + n]) before the rounding."""
    T, H, K = x.shape
    N = w.shape[1]
    _check(x, "x"); _check(w, "per-head weights"); _check(y, "y")
    if tuple(w.shape) != (H, N, K) or tuple(y.shape) != (T, H, N):
        raise KernelError(f"per-head product shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] != H * N):
        raise KernelError("the gate must be float32 [T, heads * N] with unit column stride")
    if (x.dtype == w.dtype == y.dtype == torch.bfloat16 and K % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        _call("lb_gemm_heads_mma", y.data_ptr(), x.data_ptr(), w.data_ptr(), H, T, N, K, H * K, H * N, K, N * K, N, _ptr(gate),
              gate.stride(0) if gate is not None else 0, stream)
        return
    _call("lb_gemm_plain_batched", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), dtype_code(x.dtype), w.data_ptr(),
          dtype_code(w.dtype), H, T, N, K, H * K, H * N, K, N * K, N, _ptr(gate), gate.stride(0) if gate is not None else 0, stream)


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                eps: float, stream: int, rows: torch.Tensor | None = None) -> None:
    """residual += delta (when rows is None); out = rmsnorm(residual [+ delta]) * weight, on `rows` if given."""
    _check(out, "norm output"); _check(residual, "residual", torch.float32); _check(weight, "norm weight", torch.float32)
    n = out.shape[0]
    H = out.shape[-1]
    if delta is not None:
        _check(delta, "delta")
    if rows is not None:
        _check(rows, "row index", torch.int32)
    _call("lb_add_rmsnorm", out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(), _ptr(delta),
          dtype_code(delta.dtype) if delta is not None else F32, weight.data_ptr(), _ptr(rows), n, H, eps, stream)


def rope_kv(q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor, q_out: torch.Tensor,
            positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, eps: float, stream: int,
            q_norm_w: torch.Tensor | None = None, k_norm_w: torch.Tensor | None = None,
            inv_freq: torch.Tensor | None = None, rot_dim: int = 0,
            k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
            token_seq: torch.Tensor | None = None, block_table: torch.Tensor | None = None, page_size: int = 0,
            k_out: torch.Tensor | None = None, v_out: torch.Tensor | None = None, v_dim: int = 0, rot_scale: float = 1.0) -> None:
    """Per-head norm of q and k, rotation, and the write of k and v into pages (or into k_out, v_out).

    q_in, k_in and v_in are 2-d views whose rows may be column ranges of one wider matrix; they may be float32 where
    the heads are stored in bfloat16 (a product with 32-bit output).  `v_dim`: the size of a value head if it is not
    head_dim (the value pool then has rows of that size).  `rot_scale` multiplies the rotation's sines and cosines."""
    T = q_in.shape[0]
    dt = q_out.dtype
    for t, w in ((q_in, "q"), (k_in, "k"), (v_in, "v")):
        if not t.is_cuda or t.dtype != q_in.dtype or t.stride(-1) != 1:
            raise KernelError(f"{w} must be on the GPU, of one type, with unit stride in its last dimension")
    _check(q_out, "q output", dt); _check(positions, "positions", torch.int32)
    max_pages = 0
    if k_cache is not None:
        _check(k_cache, "k pool", dt); _check(v_cache, "v pool", dt)
        _check(token_seq, "token map", torch.int32); _check(block_table, "block table", torch.int32)
        max_pages = block_table.shape[1]
    _call("lb_rope_kv", dtype_code(dt), q_in.data_ptr(), k_in.data_ptr(), v_in.data_ptr(), q_in.stride(0),
          k_in.stride(0), v_in.stride(0), q_out.data_ptr(), _ptr(k_out), _ptr(v_out), _ptr(k_cache), _ptr(v_cache),
          positions.data_ptr(), _ptr(token_seq), _ptr(block_table), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
          T, num_q_heads, num_kv_heads, head_dim, rot_dim, page_size, max_pages, eps, dtype_code(q_in.dtype), v_dim, float(rot_scale), stream)


def rotate_rows(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, head_dim: int, rot_dim: int, ranges,
                stream: int, rot_scale: float = 1.0) -> None:
    """Rotation in place of 32-bit rows: `ranges` is one or two (first column, heads, scale); each range holds `heads`
    heads of `head_dim` whose first rot_dim entries are rotated (halves paired, angle position * inv_freq[i], sines
    and cosines times rot_scale) and whose every entry is then multiplied by `scale`."""
    _rows32(x, "rows to rotate"); _check(positions, "positions", torch.int32)
    if inv_freq is not None:
        _check(inv_freq, "frequencies", torch.float32)
    rs = list(ranges)
    if not 1 <= len(rs) <= 2 or any(c < 0 or c + h * head_dim > x.shape[1] for c, h, _ in rs):
        raise KernelError("one or two column ranges inside the rows")
    (c0, h0, s0), (c1, h1, s1) = rs[0], (rs[1] if len(rs) > 1 else (0, 0, 1.0))
    _call("lb_rotate_rows", x.data_ptr(), x.stride(0), x.shape[0], positions.data_ptr(), _ptr(inv_freq), head_dim, rot_dim,
          float(rot_scale), c0, h0, float(s0), c1, h1, float(s1), stream)


def round_cols(out: torch.Tensor, x: torch.Tensor, stream: int) -> None:
    """out (contiguous, any type) = the 32-bit rows x (a column range allowed), rounded."""
    _check(out, "rounded copy"); _rows32(x, "rows to round")
    if out.shape != x.shape:
        raise KernelError("a rounded copy has its source's shape")
    _call("lb_round_cols", out.data_ptr(), dtype_code(out.dtype), x.data_ptr(), x.stride(0), x.shape[0], x.shape[1], stream)


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, token_seq: torch.Tensor, block_table: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                    stream: int, v_dim: int = 0, slopes: torch.Tensor | None = None, softcap: float = 0.0,
                    sinks: torch.Tensor | None = None, pool: int = 0, pool_k: torch.Tensor | None = None,
                    pool_v: torch.Tensor | None = None, pool_table: torch.Tensor | None = None, chunk: int = 0) -> None:
    """`chunk` = C > 0: the query at position i sees the keys floor(i / C) * C .. i only.
    `v_dim`: the size of a value head if it is not head_dim (out is then [T, heads, v_dim]); `slopes` (float32
    [heads]): the score of key j for the query at position i is lowered by slopes[h] * (i - j).  `softcap` > 0: scores
    become softcap * tanh(score / softcap).  `sinks` (float32 [heads]): exp(sinks[h]) joins the softmax's denominator.
    `pool` = P > 0 with a window: the query at i also sees entry b of the pooled cache (pool_k, pool_v through
    pool_table, one entry for every P tokens) for every b with (b + 1) P - 1 <= i - window."""
    dt = q.dtype
    if sinks is not None:
        _check(sinks, "sinks", torch.float32)
    if pool:
        _check(pool_k, "pooled k", dt); _check(pool_v, "pooled v", dt); _check(pool_table, "pooled block table", torch.int32)
    if slopes is not None:
        _check(slopes, "distance slopes", torch.float32)
    _check(q, "q"); _check(out, "attention output", dt); _check(k_cache, "k pool", dt); _check(v_cache, "v pool", dt)
    _check(positions, "positions", torch.int32); _check(token_seq, "token map", torch.int32)
    _check(block_table, "block table", torch.int32)
    _call("lb_attention_plain", dtype_code(dt), q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), q.shape[0], num_q_heads, num_kv_heads,
          head_dim, page_size, block_table.shape[1], window, scale, v_dim, _ptr(slopes), softcap, _ptr(sinks), pool,
          _ptr(pool_k) if pool else None, _ptr(pool_v) if pool else None, _ptr(pool_table) if pool else None,
          pool_table.shape[1] if pool else 0, int(chunk), stream)


def _rows32(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be float32 rows on the GPU with unit column stride")


def short_conv(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor | None,
               step, stream: int, act: bool = True) -> None:
    """out_t = act(bias + sum_j weight[j, :] * x_(t - taps + 1 + j)) over each sequence's tokens in order (weight
    [taps, channels] float32, oldest tap first; act: silu); x and out are float32 rows [T, channels] that may be column
    ranges of wider matrices; what lies before a portion is read from state[slot] ([taps - 1, channels] float32).  The
    state is not changed."""
    _rows32(out, "convolution output"); _rows32(x, "convolution input"); _check(weight, "taps", torch.float32)
    T, C = x.shape
    taps = weight.shape[0]
    if weight.shape[1] != C or tuple(out.shape) != (T, C):
        raise KernelError(f"the taps are {tuple(weight.shape)} for rows of {C}, the output {tuple(out.shape)}")
    if bias is not None:
        _check(bias, "convolution bias", torch.float32)
    if state is not None:
        _check(state, "convolution state", torch.float32)
    _call("lb_short_conv", out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), _ptr(state),
          step.token_seq.data_ptr(), step.cu_tokens.data_ptr(), step.state_slots.data_ptr(), T, C, taps, 1 if act else 0, stream)


def short_conv_state(state: torch.Tensor, x: torch.Tensor, taps: int, step, stream: int) -> None:
    """state[slot] = the last taps - 1 rows of (state[slot] ++ this step's rows of the sequence); float32."""
    _check(state, "convolution state", torch.float32); _rows32(x, "convolution input")
    _call("lb_short_conv_state", state.data_ptr(), x.data_ptr(), x.stride(0), step.cu_tokens.data_ptr(),
          step.state_slots.data_ptr(), step.num_seqs, x.shape[1], taps, stream)


def state_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None,
                     A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor | None, state: torch.Tensor, out: torch.Tensor,
                     step, heads: int, groups: int, dim: int, vdim: int, stream: int, delta: bool, unit_norm: bool = False,
                     q_scale: float = 1.0, unit_eps: float = 1e-6, rows_decay: bool = False, by_shape: bool = False) -> None:
    """A recurrence with a decay and a write strength per token over this step's tokens (csrc/state_recurrence.cu):
    delta=True the gated delta rule (b: beta's input), else the state space of Mamba-2 (k = B, q = C, v = x, a = dt's
    input, D optional).  q, k [T, groups * dim], v [T, heads * vdim], a, b [T, heads]: float32 rows, column ranges allowed;
    state [slots + 1, heads, dim, vdim] float32 is read and written at each sequence's slot; out [T, heads * vdim] float32.
    `rows_decay` (delta rule only): a decay for every row of the state; a is then [T, heads * dim] and dt_bias [heads * dim], and
    a is overwritten with the decays (one pass over it before the recurrence, so that the CTAs that share a head do not each
    form them again on the path from token to token).  `by_shape`: the kernel's layout may follow the step's shape (steps of
    single tokens keep sixteen state rows a lane, which issues fewer instructions; all others eight, which shortens the path
    from token to token); a column's terms are then added in an order that depends on the step.  Without it one layout
    serves every step, so a 32-bit result does not depend on how a sequence was cut."""
    for t, w in ((q, "q"), (k, "k"), (v, "v"), (a, "a")) + (((b, "b"),) if b is not None else ()):
        _rows32(t, w)
    _rows32(out, "recurrence output")
    _check(A_log, "A_log", torch.float32); _check(dt_bias, "dt_bias", torch.float32); _check(state, "recurrent state", torch.float32)
    if D is not None:
        _check(D, "D", torch.float32)
    T = q.shape[0]
    if (tuple(q.shape) != (T, groups * dim) or tuple(k.shape) != (T, groups * dim) or tuple(v.shape) != (T, heads * vdim)
            or tuple(a.shape) != (T, heads * dim if rows_decay else heads) or dt_bias.numel() != (heads * dim if rows_decay else heads)
            or tuple(out.shape) != (T, heads * vdim) or tuple(state.shape[1:]) != (heads, dim, vdim)):
        raise KernelError("the recurrence's operands do not fit its head counts and sizes")
    if rows_decay:
        _call("lb_channel_decay", a.data_ptr(), a.stride(0), A_log.data_ptr(), dt_bias.data_ptr(), T, heads, dim, stream)
    _call("lb_state_recurrence", 1 if delta else 0, q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
          a.data_ptr(), a.stride(0), _ptr(b), b.stride(0) if b is not None else 0, A_log.data_ptr(), dt_bias.data_ptr(), _ptr(D),
          state.data_ptr(), out.data_ptr(), out.stride(0), step.cu_tokens.data_ptr(), step.state_slots.data_ptr(), step.num_seqs,
          heads, groups, dim, vdim, 1 if unit_norm else 0, q_scale, unit_eps, 1 if T == step.num_seqs else 0, 1 if rows_decay else 0,
          1 if (by_shape and (T == step.num_seqs or _recurrence_fills_sms(step.num_seqs, heads, dim, vdim))) else 0, stream)


def _recurrence_fills_sms(num_seqs: int, heads: int, dim: int, vdim: int, sms: int = 148) -> bool:
    """Whether a step's recurrence has more CTAs than the GPU has SMs already with sixteen state rows a lane (32 value columns
    a CTA for up to 64 rows, else 16): then the instructions issued bound it, not the path from token to token."""
    cols = 32 if dim <= 64 else 16
    return num_seqs * heads * -(-vdim // cols) > sms


def gated_group_norm(out: torch.Tensor, y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor | None, groups: int, eps: float,
                     stream: int, gate_first: bool = False, act: str = "silu", scale: float = 1.0) -> None:
    """The norm behind a recurrence, in `groups` equal parts of a row, with a gate: out = y / rms_part(y) * w * act(gate),
    or with gate_first z = y * act(gate), out = z / rms_part(z) * w.  y, gate: float32 rows (column ranges allowed); weight
    float32 of the row's size, or of a part's size (then shared by the parts), or None for a norm without one; out rows of
    any type.  y may also be [planes, T, n] (contiguous): the sum of the planes, added in order, is meant."""
    planes, plane = 1, 0
    if y.dim() == 3:
        _check(y, "norm input", torch.float32)
        planes, plane = y.shape[0], y.shape[1] * y.shape[2]
        y = y[0]
    _rows32(y, "norm input"); _rows32(gate, "gate")
    if weight is not None:
        _check(weight, "norm weight", torch.float32)
    T, n = y.shape
    if (out.stride(1) != 1 or tuple(out.shape) != (T, n) or tuple(gate.shape) != (T, n) or n % groups
            or (weight is not None and weight.numel() not in (n, n // groups))):
        raise KernelError("the gated norm's operands do not fit")
    _call("lb_gated_group_norm", out.data_ptr(), dtype_code(out.dtype), out.stride(0), y.data_ptr(), y.stride(0), gate.data_ptr(),
          gate.stride(0), _ptr(weight), weight.numel() if weight is not None else 0, T, n, groups, 1 if gate_first else 0,
          {"silu": 0, "sigmoid": 1}[act], eps, scale, planes, plane, stream)


def bias_rmsnorm_cols(x: torch.Tensor, ranges, eps: float, stream: int) -> None:
    """In place on float32 rows: for each of up to three (first column, size, bias or None, norm weight or None):
    x[:, range] += bias, then, with a weight, the RMS norm over the whole range times the weight."""
    _rows32(x, "rows")
    n = len(ranges)
    if not 1 <= n <= 3:
        raise KernelError("one to three column ranges")
    for _, _, b, w in ranges:
        for t in (b, w):
            if t is not None:
                _check(t, "bias or weight", torch.float32)
    cols = (c_int * 3)(*[r[0] for r in ranges])
    sizes = (c_int * 3)(*[r[1] for r in ranges])
    biases = (c_void_p * 3)(*[_ptr(r[2]) for r in ranges])
    weights = (c_void_p * 3)(*[_ptr(r[3]) for r in ranges])
    _call("lb_bias_rmsnorm_cols", x.data_ptr(), x.stride(0), x.shape[0], n, cols, sizes, biases, weights, eps, stream)


def pool_kv(k_cache: torch.Tensor, v_cache: torch.Tensor, table: torch.Tensor, pool_k: torch.Tensor, pool_v: torch.Tensor,
            pool_table: torch.Tensor, step, num_kv_heads: int, head_dim: int, v_dim: int, page_size: int, pool: int,
            stream: int) -> None:
    """The mean key and value of every block of `pool` tokens that this step completes, from the pages into the pooled
    cache (entry b of a sequence at place b of its pooled block table)."""
    dt = k_cache.dtype
    _check(k_cache, "k pool", dt); _check(v_cache, "v pool", dt); _check(pool_k, "pooled k", dt); _check(pool_v, "pooled v", dt)
    _check(table, "block table", torch.int32); _check(pool_table, "pooled block table", torch.int32)
    _call("lb_pool_kv", dtype_code(dt), k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.shape[1], pool_k.data_ptr(),
          pool_v.data_ptr(), pool_table.data_ptr(), pool_table.shape[1], step.cu_tokens.data_ptr(), step.context_lens.data_ptr(),
          step.num_seqs, step.max_q_len // pool + 1, num_kv_heads, head_dim, v_dim, page_size, pool, stream)


def add_rmsnorm_pair(out_a: torch.Tensor, out_b: torch.Tensor | None, residual: torch.Tensor, deltas: tuple, w_a: torch.Tensor,
                     w_b: torch.Tensor | None, eps: float, stream: int) -> None:
    """residual += the deltas (none, one or two, of one type); out_a = rmsnorm(residual) * w_a and, if given,
    out_b = rmsnorm(residual) * w_b: two norms of one stream that differ in their weights."""
    _check(out_a, "norm output"); _check(residual, "residual", torch.float32); _check(w_a, "norm weight", torch.float32)
    ds = [d for d in deltas if d is not None]
    if len(ds) > 2 or any(d.dtype != ds[0].dtype for d in ds):
        raise KernelError("at most two deltas, of one type")
    for d in ds:
        _check(d, "delta")
    if out_b is not None:
        _check(out_b, "second norm output", out_a.dtype); _check(w_b, "second norm weight", torch.float32)
    _call("lb_add_rmsnorm_pair", out_a.data_ptr(), _ptr(out_b), dtype_code(out_a.dtype), residual.data_ptr(),
          ds[0].data_ptr() if ds else None, ds[1].data_ptr() if len(ds) > 1 else None, dtype_code(ds[0].dtype) if ds else F32,
          w_a.data_ptr(), _ptr(w_b), out_a.shape[0], out_a.shape[1], eps, stream)


def rmsnorm_mix2(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, w_a: torch.Tensor, w_b: torch.Tensor, sa: float, sb: float,
                 eps: float, stream: int) -> None:
    """out = sa * rmsnorm(a) * w_a + sb * rmsnorm(b) * w_b, float32 rows."""
    for t in (out, a, b, w_a, w_b):
        _check(t, "operand of the normed sum", torch.float32)
    _call("lb_rmsnorm_mix2", out.data_ptr(), a.data_ptr(), b.data_ptr(), w_a.data_ptr(), w_b.data_ptr(), sa, sb, a.shape[0],
          a.shape[1], eps, stream)


# Activations of a feed-forward without a gate (csrc/swiglu.cu, lb_activation).
PLAIN_ACTS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "xielu": 4, "relu2": 5}         # relu2: the square of relu


def activation(out: torch.Tensor, x: torch.Tensor, act: str, stream: int, p0: float = 0.0, p1: float = 0.0) -> None:
    """out = act(x) (see PLAIN_ACTS; xielu takes its two positive numbers a_p, a_n as p0, p1); x rows may be a column range."""
    _check(out, "activation output", x.dtype)
    if x.stride(1) != 1 or out.shape != x.shape:
        raise KernelError("the activation's input needs unit column stride and the output's shape")
    _call("lb_activation", dtype_code(out.dtype), out.data_ptr(), x.data_ptr(), x.stride(0), x.shape[0], x.shape[1], PLAIN_ACTS[act],
          p0, p1, stream)


# Activations of a gated feed-forward, out = act(gate) * up: silu, relu, the tanh form of gelu, and "clamped_swish",
# which clamps first (g' = min(gate, limit), u' = clamp(up, -limit, limit)) and is g' * sigmoid(1.702 g') * (u' + 1).
GATE_ACTS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "clamped_swish": 3}


def swiglu(out: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, stream: int, act: str = "silu", limit: float = 0.0) -> None:
    """out = act(gate) * up (see GATE_ACTS); gate and up are 2-d views with the same row stride."""
    if gate.stride(0) != up.stride(0) or gate.stride(1) != 1 or up.stride(1) != 1:
        raise KernelError("gate and up need the same row stride and unit column stride")
    _check(out, "swiglu output", gate.dtype)
    T, inter = out.shape
    _call("lb_swiglu", dtype_code(out.dtype), out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.stride(0), T, inter,
          GATE_ACTS[act], limit, stream)


def gemm_plain(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int) -> None:
    """y[M, N] = x[M, K] . w[N, K]^T on the 32-bit pipes; x and y may be row-strided views."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.stride(1) != 1 or y.stride(1) != 1 or not w.is_contiguous() or not (x.is_cuda and w.is_cuda and y.is_cuda):
        raise KernelError("gemm operands must be on the GPU with unit column stride; w contiguous")
    _call("lb_gemm_plain", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), dtype_code(x.dtype), w.data_ptr(),
          dtype_code(w.dtype), M, N, K, x.stride(0) if M > 1 else K, y.stride(0) if M > 1 else N, stream)


def sample(tokens: torch.Tensor, logits: torch.Tensor, stream: int, temperature: torch.Tensor | None = None,
           keys: torch.Tensor | None = None, counters: torch.Tensor | None = None) -> None:
    """tokens[r] = greedy or temperature sample of logits[r, :]; see sampling/sampler.py for the key."""
    _check(tokens, "token output", torch.int32); _check(logits, "logits", torch.float32)
    if temperature is not None:
        _check(temperature, "temperature", torch.float32); _check(keys, "keys", torch.int64)
        _check(counters, "counters", torch.int32)
    R, V = logits.shape
    _call("lb_sample", tokens.data_ptr(), logits.data_ptr(), _ptr(temperature), _ptr(keys), _ptr(counters), R, V, stream)


_WORKSPACE_ELEMS = 16 * 1024 * 1024      # float32 partials of split products (64 MB)
_COUNTERS = 4096
_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def _gemm_scratch(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Per device: the workspace for partial sums of split products and the tile counters (zero between launches)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    s = _scratch.get(key)
    if s is None:
        s = (torch.empty(_WORKSPACE_ELEMS, dtype=torch.float32, device=device),
             torch.zeros(_COUNTERS, dtype=torch.int32, device=device))
        _scratch[key] = s
    return s


def gemm_tcgen05_ok(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """The conditions of the tensor-core kernel: bfloat16 operands, K a multiple of 8, 16-byte alignment."""
    K = x.shape[1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and y.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and (x.shape[0] == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and w.is_contiguous() and x.stride(1) == 1 and y.stride(1) == 1)


class LbRowScale(ctypes.Structure):
    """Mirror of RowScale in csrc/gemm_tcgen05.cu."""
    _fields_ = [("on", c_int), ("tiles", c_int), ("sumsq", c_void_p), ("inv_width", c_float), ("eps", c_float)]


def _row_scale(sumsq: torch.Tensor | None, width: int, eps: float):
    """The argument for rows that lack their norm's factor: None, or a reference to an LbRowScale."""
    if sumsq is None:
        return None
    _check(sumsq, "partial sums of squares", torch.float32)
    return ctypes.byref(LbRowScale(1, sumsq.shape[1], sumsq.data_ptr(), 1.0 / width, eps))


def gemm_tcgen05(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int, force_bt: int = 0,
                 force_splits: int = 0, swiglu: bool = False, sumsq: torch.Tensor | None = None, eps: float = 0.0,
                 act: str = "silu", limit: float = 0.0) -> None:
    """y[M, N] = x[M, K] . w[N, K]^T on the tensor cores (tcgen05, accumulators in tensor memory).

    With `swiglu` the rows of w alternate in blocks of 64 between gate rows and up rows of the same 64
    features (see interleave_gate_up), and y[M, N/2] = act(x . gate^T) * (x . up^T), formed in the epilogue
    (act: one of GATE_ACTS; `limit` is the clamp of "clamped_swish").
    With `sumsq` [M, tiles] the rows of x lack the factor of an RMSNorm over K values: row m of the product is
    multiplied by rsqrt(sum(sumsq[m]) / K + eps), before the activation if there is one (see gemm_tcgen05_addnorm)."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N // 2 if swiglu else N):
        raise KernelError(f"gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if not gemm_tcgen05_ok(y, x, w):
        raise KernelError("gemm_tcgen05 takes bfloat16 operands with K a multiple of 8, 16-byte aligned, unit column stride")
    ws, counters = _gemm_scratch(x.device)
    _call("lb_gemm_tcgen05", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), w.data_ptr(), M, N, K,
          x.stride(0) if M > 1 else K, y.stride(0) if M > 1 else y.shape[1], ws.data_ptr(), ws.numel(), counters.data_ptr(),
          counters.numel(), force_bt, force_splits, (1 + GATE_ACTS[act]) if swiglu else 0, _row_scale(sumsq, K, eps), limit, stream)


class LbHeadEpilogue(ctypes.Structure):
    """Mirror of HeadEpilogue in csrc/gemm_tcgen05.cu."""
    _fields_ = [("on", c_int), ("num_q_heads", c_int), ("num_kv_heads", c_int), ("page_size", c_int), ("max_pages", c_int),
                ("eps", c_float), ("positions", c_void_p), ("token_seq", c_void_p), ("block_table", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("inv_freq", c_void_p), ("q_out", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p)]


def gemm_tcgen05_heads_sizes_ok(M: int, N: int, K: int, head_dim: int) -> bool:
    """The sizes the q|k|v product with the head epilogue takes (heads of 128, at most 32 tokens, a split product)."""
    lib = library()
    lib.lb_gemm_tcgen05_heads_ok.argtypes = [c_int, c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_heads_ok.restype = c_int
    return bool(lib.lb_gemm_tcgen05_heads_ok(M, N, K, head_dim))


def gemm_tcgen05_heads_ok(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int | None) -> bool:
    """The conditions of the q|k|v product whose epilogue norms, rotates and stores the heads: bfloat16, heads of
    128 rotated whole (or not at all), at most 32 tokens, a product that is split over a cluster."""
    lib = library()
    lib.lb_gemm_tcgen05_heads_ok.argtypes = [c_int, c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_heads_ok.restype = c_int
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.stride(1) == 1
            and (M == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and rot_dim in (None, head_dim) and bool(lib.lb_gemm_tcgen05_heads_ok(M, w.shape[0], K, head_dim)))


def gemm_tcgen05_addnorm_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The conditions of the product whose epilogue adds to the residual stream: bfloat16, 16-byte alignment, and sizes
    for which the product is split over a thread-block cluster (few tokens, fewer output tiles than SMs)."""
    lib = library()
    lib.lb_gemm_tcgen05_addnorm_ok.argtypes = [c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_addnorm_ok.restype = c_int
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.stride(1) == 1
            and (M == 1 or x.stride(0) % 8 == 0) and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib.lb_gemm_tcgen05_addnorm_ok(M, w.shape[0], K)))


def gemm_tcgen05_addnorm_tiles(M: int, N: int, K: int) -> int:
    """Columns of the partial sums of squares that gemm_tcgen05_addnorm writes for these sizes: blocks of 128 features
    with few tokens, the feature tiles the many-token product chooses otherwise (0: sizes it does not take)."""
    lib = library()
    lib.lb_gemm_tcgen05_addnorm_tiles.argtypes = [c_int, c_int, c_int]
    lib.lb_gemm_tcgen05_addnorm_tiles.restype = c_int
    return int(lib.lb_gemm_tcgen05_addnorm_tiles(M, N, K))


def gemm_tcgen05_addnorm(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor,
                         sumsq: torch.Tensor, stream: int) -> None:
    """residual += x . w^T; out = (residual * norm_w) rounded to bfloat16, without the factor rsqrt(mean(residual^2) + eps)
    of the RMSNorm; sumsq[m, t] = sum of residual[m]^2 over the t-th block of features (gemm_tcgen05_addnorm_tiles says
    how many blocks these sizes have).  The product that reads
    `out` is given `sumsq` and multiplies its sums by the row's factor (a row's factor commutes with a linear map), so
    the add, the copy and the norm between two products cost no kernel of their own."""
    M, K = x.shape
    N = w.shape[0]
    _check(w, "w", torch.bfloat16); _check(residual, "residual", torch.float32); _check(norm_w, "norm weight", torch.float32)
    _check(out, "normed output", torch.bfloat16); _check(sumsq, "partial sums of squares", torch.float32)
    if tuple(residual.shape) != (M, N) or tuple(out.shape) != (M, N) or sumsq.shape[0] != M or norm_w.shape[0] != N:
        raise KernelError(f"gemm_tcgen05_addnorm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, residual {tuple(residual.shape)}, sumsq {tuple(sumsq.shape)}")
    _call("lb_gemm_tcgen05_addnorm", x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0) if M > 1 else K, residual.data_ptr(),
          norm_w.data_ptr(), out.data_ptr(), sumsq.data_ptr(), sumsq.shape[1], stream)


def gemm_tcgen05_heads(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                       block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_q_heads: int,
                       num_kv_heads: int, page_size: int, eps: float, stream: int, q_norm_w: torch.Tensor | None = None,
                       k_norm_w: torch.Tensor | None = None, inv_freq: torch.Tensor | None = None,
                       sumsq: torch.Tensor | None = None, row_eps: float = 0.0) -> None:
    """x . w^T for w = [q | k | v] rows with heads of 128, finished per head in the product's epilogue: RMSNorm of
    query and key heads, rotation, queries to q_out [M, nq, 128], keys and values into their cache pages.
    `sumsq`, `row_eps`: the rows of x lack their norm's factor (see gemm_tcgen05)."""
    M, K = x.shape
    _check(x, "x", torch.bfloat16); _check(w, "w", torch.bfloat16); _check(q_out, "q output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(token_seq, "token map", torch.int32)
    _check(block_table, "block table", torch.int32)
    for t, what in ((q_norm_w, "q norm weight"), (k_norm_w, "k norm weight"), (inv_freq, "rotary table")):
        if t is not None:
            _check(t, what, torch.float32)
    he = LbHeadEpilogue(1, num_q_heads, num_kv_heads, page_size, block_table.shape[1], eps, positions.data_ptr(),
                        token_seq.data_ptr(), block_table.data_ptr(), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(inv_freq),
                        q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr())
    _call("lb_gemm_tcgen05_heads", x.data_ptr(), w.data_ptr(), M, w.shape[0], K, x.stride(0) if M > 1 else K,
          ctypes.byref(he), _row_scale(sumsq, K, row_eps), stream)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows 0..63 | up rows 0..63 | gate rows 64..127 | up rows 64..127 | ...]: the row order the
    fused SwiGLU epilogue of gemm_tcgen05 expects.  The number of rows must be a multiple of 64."""
    I, K = gate.shape
    if up.shape != gate.shape or I % 64:
        raise KernelError(f"gate and up must have the same shape with a multiple of 64 rows, got {tuple(gate.shape)}, {tuple(up.shape)}")
    return torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()


def layernorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float, stream: int, rows: torch.Tensor | None = None) -> None:
    """out[i] = (x[r] - mean) / sqrt(var + eps) * weight for r = rows[i] (or i), var the mean of the squared deviations;
    x float32."""
    _check(out, "norm output"); _check(x, "norm input", torch.float32); _check(weight, "norm weight", torch.float32)
    if rows is not None:
        _check(rows, "row index", torch.int32)
    _call("lb_layernorm", out.data_ptr(), dtype_code(out.dtype), x.data_ptr(), weight.data_ptr(), _ptr(rows), out.shape[0],
          out.shape[-1], eps, stream)


def layernorm_add(residual: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None, sa: float, sb: float, weight: torch.Tensor,
                  mult: float, eps: float, stream: int, copy: torch.Tensor | None = None) -> None:
    """residual += mult * layernorm(sa * a [+ sb * b]) * weight, in 32-bit; `copy`, if given, receives the new residual
    rounded to its type."""
    _check(residual, "residual", torch.float32); _check(a, "sublayer output"); _check(weight, "norm weight", torch.float32)
    if b is not None:
        _check(b, "second sublayer output", a.dtype)
    if a.shape != residual.shape or (b is not None and b.shape != a.shape) or (copy is not None and copy.shape != residual.shape):
        raise KernelError("the sublayer outputs and the copy must have the residual's shape")
    if copy is not None:
        _check(copy, "residual copy")
    _call("lb_layernorm_add", residual.data_ptr(), a.data_ptr(), _ptr(b), dtype_code(a.dtype), sa, sb, weight.data_ptr(), mult, eps,
          _ptr(copy), dtype_code(copy.dtype) if copy is not None else F32, residual.shape[0], residual.shape[1], stream)


def round_copy(out: torch.Tensor, x: torch.Tensor, stream: int) -> None:
    """out = x (float32) rounded to out's type."""
    _check(out, "copy"); _check(x, "source", torch.float32)
    if out.shape != x.shape:
        raise KernelError("a rounded copy has its source's shape")
    _call("lb_round_copy", out.data_ptr(), dtype_code(out.dtype), x.data_ptr(), x.numel(), stream)


def decay_row_split(num_seqs: int, heads: int, dim: int, vdim: int, max_tokens_a_seq: int) -> int:
    """Into how many shares of rows the kernel that forms outputs side by side cuts a head's state for a step of this
    shape (0: the step runs token by token): as many as fill the SMs, with 32 to 256 rows a share."""
    lib = library()
    lib.lb_decay_row_split.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.lb_decay_row_split.restype = c_int
    return int(lib.lb_decay_row_split(num_seqs, heads, dim, vdim, max_tokens_a_seq))


def decay_recurrence(pre: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
                     out: torch.Tensor, step, heads: int, dim: int, vdim: int, stream: int, max_tokens_a_seq: int = 0,
                     row_split: int = 0, act: bool = True) -> None:
    """Linear attention with a fixed decay per head over this step's tokens: S <- decay_h S + k v^T, out = S^T q with
    q, k, v = silu of the columns of `pre` (float32, row-strided) at q_col, k_col, v_col (act=False: the columns as they are); state [slots + 1, heads, dim, vdim]
    float32 is read and written at each sequence's slot; out [T, heads * vdim] float32.
    `row_split` >= 1 (see decay_row_split): the outputs of 16 tokens at a time are formed from the state before them
    and the tokens' own scores (32-bit, outputs equal within rounding, several times faster), the state's rows shared out
    over row_split CTAs; out is then [row_split, T, heads * vdim] and the sum over its first dimension is meant.
    With 0 every output's sum has one order however the sequence is cut."""
    _check(decay, "decay", torch.float32); _check(state, "recurrent state", torch.float32); _check(out, "recurrence output", torch.float32)
    if pre.dtype != torch.float32 or pre.stride(1) != 1 or not pre.is_cuda:
        raise KernelError("the input projections must be float32 on the GPU with unit column stride")
    T = pre.shape[0]
    if tuple(out.shape) != ((row_split, T, heads * vdim) if row_split >= 1 else (T, heads * vdim)):
        raise KernelError(f"the recurrence's output has the wrong shape {tuple(out.shape)}")
    _call("lb_decay_recurrence", pre.data_ptr(), pre.stride(0), q_col, k_col, v_col, decay.data_ptr(), state.data_ptr(),
          out.data_ptr(), step.cu_tokens.data_ptr(), step.state_slots.data_ptr(), step.num_seqs, heads, dim, vdim,
          max_tokens_a_seq, row_split, T * heads * vdim, 1 if act else 0, stream)


def rmsnorm_gated(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, scale: float, eps: float,
                  stream: int) -> None:
    """out = x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate) * scale, row by row; x float32 [T, n] contiguous (or
    [planes, T, n], whose sum over the planes is meant), gate float32 and out (any type) may be column ranges of wider
    matrices."""
    _check(x, "norm input", torch.float32); _check(weight, "norm weight", torch.float32)
    planes = x.shape[0] if x.dim() == 3 else 1
    T, n = x.shape[-2], x.shape[-1]
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or out.stride(1) != 1 or tuple(gate.shape) != (T, n) or tuple(out.shape) != (T, n):
        raise KernelError("gate (float32) and out must be [T, n] views with unit column stride")
    _call("lb_rmsnorm_gated", out.data_ptr(), dtype_code(out.dtype), out.stride(0) if T > 1 else n, x.data_ptr(), weight.data_ptr(),
          gate.data_ptr(), gate.stride(0) if T > 1 else n, scale, eps, T, n, planes, T * n, stream)


def head_gate(out: torch.Tensor, x: torch.Tensor, gate: torch.Tensor, scale: float, stream: int) -> None:
    """out[t, h * vdim + e] = x[t, h, e] * sigmoid(gate[t, h]) * scale; x [T, heads, vdim] contiguous, gate float32 [T, heads]
    and out [T, heads * vdim] (x's type) may be column ranges of wider matrices."""
    _check(x, "heads")
    T, H, vd = x.shape
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or out.stride(1) != 1 or out.dtype != x.dtype or tuple(gate.shape) != (T, H) or tuple(out.shape) != (T, H * vd):
        raise KernelError("gate (float32 [T, heads]) and out ([T, heads * vdim], the heads' type) must have unit column stride")
    _call("lb_head_gate", out.data_ptr(), dtype_code(out.dtype), out.stride(0) if T > 1 else H * vd, x.data_ptr(), gate.data_ptr(),
          gate.stride(0) if T > 1 else H, scale, T, H, vd, stream)


def route_topk(ids: torch.Tensor, weights: torch.Tensor, logits: torch.Tensor, correction: torch.Tensor | None, groups: int,
               keep: int, scale: float, stream: int) -> None:
    """The router's choice for every token: ids [T, top] int32 and weights [T, top] float32 from logits [T, experts]
    float32 (row-strided).  Scores are sigmoid(logits); chosen are the `top` largest of score + correction among the
    experts of the `keep` best of `groups` equal groups of neighbours (a group is worth its two largest); the weights
    are the chosen plain scores over their sum (+ 1e-20), times scale."""
    _check(ids, "expert ids", torch.int32); _check(weights, "expert weights", torch.float32)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("the router's logits must be float32 with unit column stride")
    if correction is not None:
        _check(correction, "correction", torch.float32)
    T, E = logits.shape
    _call("lb_route_topk", ids.data_ptr(), weights.data_ptr(), logits.data_ptr(), logits.stride(0) if T > 1 else E, _ptr(correction),
          T, E, ids.shape[1], groups, keep, scale, stream)


def expert_tile_rows() -> int:
    lib = library()
    lib.lb_expert_tile_rows.restype = c_int
    return int(lib.lb_expert_tile_rows())


def expert_max_tiles(pairs: int, experts: int) -> int:
    """The most row tiles the experts' products can have for this many (token, choice) pairs."""
    return -(-pairs // expert_tile_rows()) + experts


def expert_dispatch(ids: torch.Tensor, experts: int, offsets: torch.Tensor, pair_at: torch.Tensor, place_of: torch.Tensor,
                    meta: torch.Tensor, stream: int) -> None:
    """Sort the (token, choice) pairs by expert, on the device: offsets [experts + 1], pair_at [pairs] (the pair at each
    place), place_of [pairs], meta [4 + 3 * expert_max_tiles] (the row tiles of the products)."""
    for t, what in ((ids, "expert ids"), (offsets, "offsets"), (pair_at, "pair list"), (place_of, "places"), (meta, "tile list")):
        _check(t, what, torch.int32)
    pairs = ids.numel()
    if offsets.numel() < experts + 1 or pair_at.numel() < pairs or place_of.numel() < pairs or meta.numel() < 4 + 3 * expert_max_tiles(pairs, experts):
        raise KernelError("expert_dispatch: an output is too small")
    _call("lb_expert_dispatch", ids.data_ptr(), pairs, experts, offsets.data_ptr(), pair_at.data_ptr(), place_of.data_ptr(),
          meta.data_ptr(), stream)


def expert_gemm(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, meta: torch.Tensor, pair_at: torch.Tensor, top: int,
                gather: bool, stream: int, act: str | None = None, limit: float = 0.0, fast: bool = True,
                interleaved: bool = False) -> None:
    """y[place] = x[row(place)] . w[e]^T for the places of every expert e (see expert_dispatch); w [experts, N, K].
    `gather`: row(place) is the pair's token, else the place.  With `act`, w[e] is N/2 gate rows then N/2 up rows (or,
    `interleaved`, blocks of 64 gate rows and their 64 up rows in turn, see interleave_gate_up) and y[place] =
    act(gate) * up with N/2 columns."""
    _check(y, "expert output"); _check(x, "expert input"); _check(w, "expert weights")
    E, N, K = w.shape
    pairs = pair_at.numel()
    cols = N // 2 if act is not None else N
    if x.shape[1] != K or y.shape[1] != cols or y.shape[0] != pairs:
        raise KernelError(f"expert_gemm shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _call("lb_expert_gemm", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), dtype_code(x.dtype), w.data_ptr(), dtype_code(w.dtype),
          meta.data_ptr(), pair_at.data_ptr(), expert_max_tiles(pairs, E), N, K, K, cols, top, 1 if gather else 0,
          1 if act is not None else 0, GATE_ACTS[act] if act is not None else 0, limit, 1 if fast else 0, 1 if interleaved else 0, stream)


GROUP_TILE = 128          # token tile of the grouped tensor-memory product


def expert_padded_places(pairs: int, experts: int) -> int:
    """Places the pairs of token and choice take when every expert's run is padded to whole tiles of GROUP_TILE."""
    return -(-(pairs + experts * (GROUP_TILE - 1)) // GROUP_TILE) * GROUP_TILE


def expert_dispatch_padded(ids: torch.Tensor, experts: int, pair_at: torch.Tensor, place_of: torch.Tensor, tile_group: torch.Tensor,
                           stream: int) -> None:
    """Sort the pairs by expert with every run padded to whole tiles: pair_at [places] (-1: padding), place_of [pairs],
    tile_group [places / GROUP_TILE] (the expert of each tile), places = expert_padded_places(pairs, experts)."""
    for t, what in ((ids, "expert ids"), (pair_at, "pair list"), (place_of, "places"), (tile_group, "tile list")):
        _check(t, what, torch.int32)
    pairs, places = ids.numel(), pair_at.numel()
    if places != expert_padded_places(pairs, experts) or place_of.numel() < pairs or tile_group.numel() < places // GROUP_TILE:
        raise KernelError("expert_dispatch_padded: an output has the wrong size")
    _call("lb_expert_dispatch_padded", ids.data_ptr(), pairs, experts, GROUP_TILE, places, pair_at.data_ptr(), place_of.data_ptr(),
          tile_group.data_ptr(), stream)


def expert_gather_rows(xs: torch.Tensor, x: torch.Tensor, pair_at: torch.Tensor, top: int, stream: int) -> None:
    """xs[place] = x[pair_at[place] // top] (zeros where the place is padding); bfloat16 rows of a multiple of 8 values."""
    _check(xs, "gathered rows", torch.bfloat16); _check(x, "rows", torch.bfloat16); _check(pair_at, "pair list", torch.int32)
    if xs.shape[0] != pair_at.numel() or xs.shape[1] != x.shape[1]:
        raise KernelError("expert_gather_rows: shapes do not fit")
    _call("lb_expert_gather_rows", xs.data_ptr(), x.data_ptr(), pair_at.data_ptr(), xs.shape[0], top, x.shape[1], stream)


def gemm_tcgen05_grouped(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, stream: int,
                         act: str | None = None, limit: float = 0.0) -> None:
    """y[m] = x[m] . w[g]^T with g = tile_group[m // GROUP_TILE], on the tensor cores (the many-token kernel of gemm_tcgen05);
    w [groups, N, K] bfloat16.  With `act`, w[g] holds gate and up rows interleaved in blocks of 64 and y = act(gate) * up."""
    _check(y, "y"); _check(x, "x", torch.bfloat16); _check(w, "grouped weights", torch.bfloat16); _check(tile_group, "tile list", torch.int32)
    G, N, K = w.shape
    M = x.shape[0]
    cols = N // 2 if act is not None else N
    if x.shape[1] != K or tuple(y.shape) != (M, cols) or tile_group.numel() * GROUP_TILE < M:
        raise KernelError(f"gemm_tcgen05_grouped shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _call("lb_gemm_tcgen05_grouped", y.data_ptr(), dtype_code(y.dtype), x.data_ptr(), w.data_ptr(), M, N, K, K, cols,
          (1 + GATE_ACTS[act]) if act is not None else 0, limit, tile_group.data_ptr(), G, stream)


def expert_combine(out: torch.Tensor, y: torch.Tensor, weights: torch.Tensor, place_of: torch.Tensor, stream: int,
                   always: torch.Tensor | None = None) -> None:
    """out[t] = sum_k weights[t, k] * y[place_of[t, k]] (+ always[t]), in 32-bit, k in order."""
    _check(out, "combined output"); _check(y, "expert outputs", torch.float32); _check(weights, "expert weights", torch.float32)
    _check(place_of, "places", torch.int32)
    if always is not None:
        _check(always, "shared expert output")
    T, W = out.shape
    _call("lb_expert_combine", out.data_ptr(), dtype_code(out.dtype), y.data_ptr(), weights.data_ptr(), place_of.data_ptr(),
          _ptr(always), dtype_code(always.dtype) if always is not None else F32, T, weights.shape[1], W, stream)


def zero_rows(state: torch.Tensor, slots: torch.Tensor, stream: int) -> None:
    """state[slots[i]] = 0 for every non-negative entry of slots (int32, on the device)."""
    _check(state, "state"); _check(slots, "slot list", torch.int32)
    row_bytes = state[0].numel() * state.element_size()
    _call("lb_zero_rows", state.data_ptr(), row_bytes, state.shape[0], slots.data_ptr(), slots.shape[0], stream)


def upload(dst_ptr: int, src_ptr: int, nbytes: int, stream: int) -> None:
    """One asynchronous copy from pinned host memory to the device, in the order of `stream`."""
    _call("lb_upload", dst_ptr, src_ptr, nbytes, stream)


def launch_count() -> int:
    """Kernels the library has launched so far in this process."""
    lib = library()
    lib.lb_launch_count.restype = c_ulonglong
    return int(lib.lb_launch_count())


def device_error() -> int:
    """Code that a kernel left when one of its bounded waits gave up (0: none).  Synchronises the device."""
    lib = library()
    lib.lb_device_error.restype = c_int
    lib.lb_attention_tcgen05_device_error.restype = c_int
    lib.lb_attention_flash_device_error.restype = c_int
    return (int(lib.lb_device_error()) or int(lib.lb_attention_tcgen05_device_error())
            or int(lib.lb_attention_flash_device_error()))


def linear(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, stream: int, fast: bool) -> None:
    """y = x . w^T.  `fast` allows the tensor-core kernel where its conditions hold (otherwise, and
    always on the 32-bit path, the product runs on the ordinary pipes)."""
    if fast and gemm_tcgen05_ok(y, x, w):
        gemm_tcgen05(y, x, w, stream)
    else:
        gemm_plain(y, x, w, stream)


_attn_ws: dict[int, torch.Tensor] = {}
_attn_ws_retired: list[torch.Tensor] = []


def _attention_workspace(device: torch.device, elems: int) -> torch.Tensor:
    """Per device: float32 scratch for the partial results of split attention; grows on demand.

    A recorded CUDA graph keeps the address of the workspace it was recorded with, so a workspace that has
    been handed out is never freed: when a larger one is needed the old one is retired, not released (it stays
    valid for the recordings that name it; launches are ordered on one stream, so sharing it is safe).  Sizes at
    least double, which bounds what the retired ones hold to the size of the current one."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < elems:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace cannot grow while a CUDA graph is captured; run the step once before")
        if ws is not None:
            _attn_ws_retired.append(ws)
        ws = torch.empty(max(elems, 1 << 20, 2 * ws.numel() if ws is not None else 0), dtype=torch.float32, device=device)
        _attn_ws[key] = ws
    return ws


def attention_flash_ok(q: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """The conditions of the tensor-core attention kernel."""
    return (q.dtype == torch.bfloat16 and head_dim % 8 == 0 and 8 <= head_dim <= 128
            and num_q_heads % num_kv_heads == 0 and num_q_heads // num_kv_heads <= 64)


def attention_splits(num_tiles: int, num_kv_heads: int, max_span: int, max_rows: int = 64, slots: int = 296,
                     wide_clusters: int = 0) -> int:
    """Into how many key ranges a launch is cut.  `slots` is how many CTAs run at a time (two on each
    of the 148 SMs).  Fewer CTAs than slots: as many ranges as still fit one wave; for tiles of up to
    16 query rows a count below 16 becomes a power of two, because up to 8 ranges of such tiles combine
    inside a thread-block cluster instead of through a workspace and a second kernel.  More CTAs than
    slots: the count (up to 8) that costs least by a model of the last wave and of the CTAs' fixed costs.  A range
    has 256 keys at least.  `wide_clusters`: how many clusters of 16 CTAs the GPU keeps resident (0: none); a launch of
    at most that many tiles x kv heads over up to 24 K keys that would take 16 or more ranges takes 16 in such clusters
    (one request of 8 kv heads at 8 K keys: 12.9 us against 17.5 us with 32 ranges through the workspace)."""
    base = max(num_tiles * num_kv_heads, 1)
    cap = max(1, min(max_span // 256, 64))
    if max_rows > 16 and base >= slots // 2:
        return 1         # portions of prompts fill the SMs by themselves; cutting them only adds partial results
    if base <= slots:
        s = max(1, min(slots // base, cap))
        if max_rows <= 16 and s < 16:
            s = 8 if s >= 8 else 4 if s >= 4 else 2 if s >= 2 else 1
        elif max_rows <= 16 and base <= wide_clusters and max_span <= 24576:
            s = 16
        return s
    # More tiles than slots.  The memory is busy as long as about half the slots are filled, so only a last wave of fewer
    # CTAs than that costs (the more the longer a CTA runs), and every CTA costs its start and its end: measured,
    # about 6 us of a slot per CTA, 0.022 us per key of a CTA's range while a full wave shares the memory.
    best, best_cost = 1, float("inf")
    for s in range(1, min(cap, 8) + 1):
        rest = (base * s) % slots
        tail = 0.6 * (0.022 * max_span / s) * max(0.0, 1.0 - rest / (slots / 2)) if rest else 0.0
        cost = 6.0 * base * s / slots + tail
        if cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


_wide_clusters: dict[int, int] = {}


def attention_wide_clusters(head_dim: int) -> int:
    """How many clusters of 16 CTAs of the decode attention kernel the GPU keeps resident at a time (0: it does not
    schedule clusters of that size)."""
    key = 64 if head_dim <= 64 else 128
    if key not in _wide_clusters:
        lib = library()
        lib.lb_attention_flash_wide_clusters.restype = c_int
        lib.lb_attention_flash_wide_clusters.argtypes = [c_int]
        _wide_clusters[key] = max(0, int(lib.lb_attention_flash_wide_clusters(key)))
    return _wide_clusters[key]


def attention_flash(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor, max_rows: int,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                    splits: int, stream: int, force_workspace: bool = False, tma: bool = True, kv_share: int = 1,
                    slopes: torch.Tensor | None = None, softcap: float = 0.0, sinks: torch.Tensor | None = None, pool: int = 0,
                    pool_k: torch.Tensor | None = None, pool_v: torch.Tensor | None = None,
                    pool_table: torch.Tensor | None = None, chunk: int = 0) -> None:
    """Tensor-core attention over pages.  tiles: int32 [n, 4] of (first token, tokens, request index, 0).
    `kv_share` > 1: the pools hold num_kv_heads / kv_share heads, and kv head j of this call reads pool head j // kv_share
    (many query heads on one cached head, cut into groups of at most 16 so that decoded tokens fit the decode kernel's tiles).
    `force_workspace` sends the partial results of the splits through the workspace and the combining
    kernel even where a cluster could combine them.  Tiles of at most 16 query rows (decoded tokens) over pages of
    8 to 128 tokens run in the kernel whose keys and values a warp of its own fetches by TMA; `tma=False` keeps them
    in the kernel that fetches with 16-byte copies, which takes every page size.  `softcap`, `sinks` and `pool` (with
    pool_k, pool_v, pool_table) and `chunk` as in attention_plain; a launch with any of them runs in the kernel with
    16-byte copies."""
    if softcap > 0 or sinks is not None or pool or chunk:
        tma = False
    if sinks is not None:
        _check(sinks, "sinks", torch.float32)
    if pool:
        _check(pool_k, "pooled k", torch.bfloat16); _check(pool_v, "pooled v", torch.bfloat16)
        _check(pool_table, "pooled block table", torch.int32)
    _check(q, "q", torch.bfloat16); _check(out, "attention output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(block_table, "block table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    n = tiles.shape[0]
    ws, ws_elems = None, 0
    by_tma = tma and max_rows <= 16 and page_size in (8, 16, 32, 64, 128)
    in_cluster = max_rows <= 16 and not force_workspace and (2 <= splits <= 8 or (splits <= 16 and by_tma))
    if splits > 1 and not in_cluster:
        ws_elems = n * num_kv_heads * splits * max_rows * (head_dim + 2)
        ws = _attention_workspace(q.device, ws_elems)
        ws_elems = ws.numel()
    _call("lb_attention_flash_ex", q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), block_table.data_ptr(), tiles.data_ptr(), n, num_q_heads, num_kv_heads, head_dim,
          page_size, block_table.shape[1], k_cache.shape[0] if tma else 0, window, scale,
          -splits if force_workspace else splits, max_rows, _ptr(ws), ws_elems, kv_share, _ptr(slopes), softcap, _ptr(sinks),
          pool, _ptr(pool_k) if pool else None, _ptr(pool_v) if pool else None, _ptr(pool_table) if pool else None,
          pool_table.shape[1] if pool else 0, int(chunk), stream)


def attention_tcgen05_ok(q: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                         max_pages: int = 0) -> bool:
    """The conditions of the tensor-memory attention kernel: bfloat16, head size 128, at most 128 query heads per
    kv head, pages of 8, 16, 32, 64 or 128 tokens, at most 4096 pages a request."""
    lib = library()
    lib.lb_attention_tcgen05_ok.restype = c_int
    return (q.dtype == torch.bfloat16 and max_pages <= 4096
            and bool(lib.lb_attention_tcgen05_ok(num_q_heads, num_kv_heads, head_dim, page_size)))


def attention_tcgen05_splits(num_tiles: int, num_kv_heads: int, max_span: int, sms: int = 148) -> int:
    """Into how many key ranges the work items of the tensor-memory kernel are cut.  A CTA takes a whole SM, so a launch
    of fewer CTAs than SMs (one portion of a few hundred tokens behind a long context) leaves SMs idle for as long as
    its longest item lasts, and one of a few more CTAs than SMs runs a second round for them.  By a model fitted to
    measurements (8 kv heads, items of 64 tokens): a CTA takes 6 us plus 0.0177 us per key it visits (8 us when it
    leaves partial results), the launch as many rounds of that as its CTAs need on the SMs, and the second kernel
    6 us plus 0.06 us per CTA (266 KB of partial results written and read again).  A cut must promise 5 % at least.  64 CTAs behind 7680 keys: 140 us whole, 87 us in two ranges; 8 CTAs behind 16 K keys:
    240 and 43 us in eight.  A range has four blocks of 64 keys at least.  The count depends on the launch's shape alone
    (tiles, kv heads, the bound of the context), never on where the requests stand, so a recorded step keeps it; it
    takes every item to see `max_span` keys, which overrates whole prompts, whose items see half of that on average,
    but those either fill the SMs many times over or are short."""
    ctas = max(num_tiles * num_kv_heads, 1)
    per_key = 0.0177 * max_span
    best, best_cost = 1, -(-ctas // sms) * (6.0 + per_key)
    for s in range(2, min(8, max_span // 256) + 1):
        cost = -(-ctas * s // sms) * (8.0 + per_key / s) + 6.0 + 0.06 * ctas * s
        if cost < 0.95 * best_cost:
            best, best_cost = s, cost
    return best


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      positions: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor, num_q_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, stream: int,
                      key_splits: int = 1, slopes: torch.Tensor | None = None) -> None:
    """Attention of portions of prompts on tcgen05 (S and O in tensor memory).  tiles: int32 [n, 4] of
    (first token, tokens, request index, 0) with tokens <= 2 * (128 // (nq // nkv)).  With key_splits > 1 the keys of
    every tile are cut into that many ranges, a CTA each, combined by a second kernel."""
    _check(q, "q", torch.bfloat16); _check(out, "attention output", torch.bfloat16)
    _check(k_cache, "k pool", torch.bfloat16); _check(v_cache, "v pool", torch.bfloat16)
    _check(positions, "positions", torch.int32); _check(block_table, "block table", torch.int32)
    _check(tiles, "tiles", torch.int32)
    ws, ws_elems = None, 0
    if key_splits > 1:
        ws = _attention_workspace(q.device, tiles.shape[0] * num_kv_heads * key_splits * 256 * (head_dim + 2))
        ws_elems = ws.numel()
    _call("lb_attention_tcgen05", q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
          positions.data_ptr(), block_table.data_ptr(), tiles.data_ptr(), tiles.shape[0], q.shape[0], num_q_heads,
          num_kv_heads, head_dim, page_size, k_cache.shape[0], block_table.shape[1], window, scale, key_splits,
          _ptr(ws), ws_elems, _ptr(slopes), stream)


def attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step, group: int,
              num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
              stream: int, plan=None, kv_share: int = 1, v_dim: int = 0, slopes: torch.Tensor | None = None,
              softcap: float = 0.0, sinks: torch.Tensor | None = None, pool: int = 0, pool_k: torch.Tensor | None = None,
              pool_v: torch.Tensor | None = None, pool_group: int = -1, chunk: int = 0) -> None:
    """Causal attention of this step's queries over the pages of their requests.  With a `plan` (tile lists
    by kind on the device, see parts/attention.py) the tensor-core kernels run where their conditions hold:
    portions of prompts go to the tcgen05 kernel, the rest (decoded tokens, short portions, other head
    sizes) to the mma.sync kernels; everything else, and every step without a plan, goes to the plain kernel.
    `kv_share` > 1: the plan's lists other than "big" were made for groups of num_q_heads / (num_kv_heads * kv_share)
    query heads, kv_share of which read one cached head (see attention_flash).  A capped score (`softcap`), sinks and
    pooled blocks behind the window (`pool` tokens a block, their means in pool_k / pool_v, pages of group `pool_group`)
    and chunks (`chunk` = C: a query sees the keys of its own run of C positions only) run in the mma.sync kernel with
    16-byte copies, for portions and for decoded tokens, or in the plain kernel."""
    extras = softcap > 0 or sinks is not None or pool > 0 or chunk > 0
    pool_table = step.block_tables[pool_group] if pool else None
    if (plan is None or (v_dim and v_dim != head_dim) or ((slopes is not None or extras) and not scale > 0)
            or (pool and kv_share != 1) or not attention_flash_ok(q, num_q_heads, num_kv_heads * kv_share, head_dim)):
        # value heads of another size than the keys' are the plain kernel's alone
        attention_plain(q, out, k_cache, v_cache, step.positions, step.token_seq, step.block_tables[group],
                        num_q_heads, num_kv_heads, head_dim, page_size, window, scale, stream, v_dim=v_dim, slopes=slopes,
                        softcap=softcap, sinks=sinks, pool=pool, pool_k=pool_k, pool_v=pool_v, pool_table=pool_table, chunk=chunk)
        return
    meta, most_rows = plan.arrays, plan.host["rows"]
    longest = step.span_hint or step.max_context_len                 # a recorded step plans for a bucket of lengths
    span = min(longest, window + step.max_q_len) if window > 0 else longest
    if chunk:
        span = min(span, chunk)
    if pool:
        span += -(-max(longest - window, 0) // pool)                 # one entry a block behind the window
    kinds = ["all"]
    if slopes is not None:
        _check(slopes, "distance slopes", torch.float32)
    if not extras and "big" in meta and attention_tcgen05_ok(q, num_q_heads, num_kv_heads, head_dim, page_size,
                                                             step.block_tables[group].shape[1]):
        attention_tcgen05(q, out, k_cache, v_cache, step.positions, step.block_tables[group], meta["big"],
                          num_q_heads, num_kv_heads, head_dim, page_size, window, scale, stream,
                          key_splits=attention_tcgen05_splits(meta["big"].shape[0], num_kv_heads, span), slopes=slopes)
        kinds = ["rest"] if "rest" in meta else []
    for kind in kinds:
        tiles = meta[kind]
        rows = min(most_rows[kind], 64)
        wide = attention_wide_clusters(head_dim) if rows <= 16 and page_size in (8, 16, 32, 64, 128) and not extras else 0
        splits = attention_splits(tiles.shape[0], num_kv_heads * kv_share, span, rows, wide_clusters=wide)
        attention_flash(q, out, k_cache, v_cache, step.positions, step.block_tables[group], tiles, rows,
                        num_q_heads, num_kv_heads * kv_share, head_dim, page_size, window, scale, splits, stream, kv_share=kv_share,
                        slopes=slopes, softcap=softcap, sinks=sinks, pool=pool, pool_k=pool_k, pool_v=pool_v, pool_table=pool_table,
                        chunk=chunk)
