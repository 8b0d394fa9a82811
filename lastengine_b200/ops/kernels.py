"""Python face of the CUDA kernels: checks shapes and types, then calls the C entry points.

Every function launches on torch's current stream and returns at once.  Tensors are only
containers here: no torch arithmetic runs on the product path.  A call on a machine without
the built library, or with tensors that are not on a CUDA device, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

from . import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_lib = None
_timer = None      # a KernelTimer while one is active


def lib():
    global _lib
    if _lib is None:
        _lib = _build.load()
        _declare(_lib)
    return _lib if _timer is None else _timer.proxy


class KernelTimer:
    """Device time of every kernel entry point called while it is active, by name.

        with kernels.KernelTimer() as t:
            engine.step(...)
        t.summary()  ->  {entry point: (calls, milliseconds)}, longest first

    Every call is bracketed by two CUDA events on the launching stream, as the reference's per-kernel
    timer does behind LE_EVT (src/gpu/dense.rs:47-51, :348-388).  An event between two kernels keeps
    the second from starting under the first (programmatic dependent launch), so the times are
    those of kernels run one after the other: they add up to more than the step takes, and their
    shares are what to read.  `head_start_ms` > 0 first occupies the device for about that long, so
    that the host has queued the step's launches before the device reaches them and no event pair
    contains the host's time between two launches.  Not for captured graphs or timed runs."""

    def __init__(self, head_start_ms: float = 0.0):
        self.head_start_ms = float(head_start_ms)
        self.events: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        real = lib()
        timer = self

        class _Proxy:
            def __getattr__(self, name):
                fn = getattr(real, name)
                if not name.startswith("leb_") or fn.argtypes is None or not fn.argtypes or fn.argtypes[-1] is not c_void_p:
                    return fn          # queries and settings: no stream, nothing to time

                def timed(*args):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    rc = fn(*args)
                    b.record()
                    timer.events.append((name, a, b))
                    return rc
                return timed
        self.proxy = _Proxy()

    def __enter__(self):
        global _timer
        if _timer is not None:
            raise KernelError("a KernelTimer is already active")
        if self.head_start_ms > 0:
            torch.cuda._sleep(int(self.head_start_ms * 1.5e6))      # cycles, at some 1.5 GHz
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None
        torch.cuda.synchronize()
        return False

    def summary(self) -> dict[str, tuple[int, float]]:
        acc: dict[str, list] = {}
        for name, a, b in self.events:
            e = acc.setdefault(name, [0, 0.0])
            e[0] += 1
            e[1] += a.elapsed_time(b)
        return {k: (v[0], v[1]) for k, v in sorted(acc.items(), key=lambda kv: -kv[1][1])}


def _declare(L) -> None:
    P, I, F, S = c_void_p, c_int, c_float, c_size_t
    sig = {
        "leb_embed": [P, P, I, P, I, I, I, F, P],
        "leb_rmsnorm": [P, I, P, P, P, I, I, F, I, P],
        "leb_swiglu": [P, I, P, I, I, I, P],
        "leb_gather_rows": [P, P, I, P, I, I, I, P],
        "leb_add": [P, P, S, P],
        "leb_shortconv": [P, P, I, P, P, P, P, P, P, P, I, I, I, I, P],
        "leb_qk_rope_store": [P, P, I, P, P, I, P, P, I, P, I, P, P, P, P, P, F, P, I, I, I, I, I, I, I, I, I, I, I, P],
        "leb_attention": [P, P, P, P, P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, I, I, P],
        "leb_gated_act": [P, I, P, I, I, I, I, F, F, P],
        "leb_layernorm": [P, I, P, P, P, I, I, F, P],
        "leb_scaled_residual": [P, P, F, P, I, P, F, I, I, P],
        "leb_latent_prep": [P, P, I, I, P, P, I, P, P, P, P, P, F, P, I, I, I, I, I, I, P],
        "leb_latent_q_split": [P, P, P, I, P, P, I, I, I, I, I, I, P],
        "leb_heads_to_rows": [P, P, I, I, I, I, P],
        "leb_latent_attention": [P, I, P, P, P, P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P],
        "leb_latent_attention_mma_supported": [I, I, I],
        "leb_gemm_bf16_any": [P, I, P, P, I, I, I, I, I, I, P, I, S, P],
        "leb_gated_residual": [P, P, P, I, I, P, P, I, P, F, I, I, P],
        "leb_stream_add": [P, P, P, I, I, P],
        "leb_causal_conv": [P, I, P, I, I, P, P, P, P, P, P, I, I, I, I, I, P],
        "leb_retention": [P, P, P, P, P, I, I, P, P, P, I, F, F, P, P, P, P, I, I, I, I, I, P],
        "leb_retention_chunked": [P, P, P, P, P, I, I, P, P, P, P, I, F, F, P, P, P, P, I, I, I, I, I, P],
        "leb_retention_chunked_supported": [I, I],
        "leb_gemm_f32": [P, P, P, I, I, I, I, I, I, P, I, S, P],
        "leb_gemm_bf16_small": [P, I, P, P, I, I, I, I, I, I, P, I, S, I, P],
        "leb_gemm_bf16_stream": [P, I, P, P, I, I, I, I, I, I, P, I, I, F, P, P, P, P],
        "leb_gemm_bf16_stream_grouped": [P, I, P, P, I, I, I, I, I, I, P, I, S, P],
        "leb_gemm_bf16_stream_conv": [P, P, P, I, I, I, I, I, P, P, P, P, P, I, P, I, I, F, P],
        "leb_gemm_bf16_tc_grouped": [P, I, P, P, I, I, I, I, I, I, P, I, P, P],
        "leb_gemm_bf16_tc2": [P, I, P, P, I, I, I, I, I, I, P, P],
        "leb_moe_router": [P, P, P, I, P, P, I, I, I, I, I, F, P],
        "leb_moe_align": [P, P, P, P, I, I, P],
        "leb_moe_combine": [P, P, P, P, I, I, I, I, P],
        "leb_penalties": [P, P, P, I, I, I, F, F, P],
        "leb_argmax": [P, P, I, I, P],
        "leb_sample": [P, P, P, I, I, I, F, F, F, P],
        "leb_advance": [P, P, P, P, P, I, P],
        "leb_feed_tokens": [P, P, P, I, P],
        "leb_penalties_slots": [P, P, P, P, I, I, I, F, F, P],
        "leb_history_append": [P, P, P, P, I, I, P],
        "leb_attention_decode_supported": [I, I, I, I],
        "leb_attention_decode": [P, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "leb_attention_merge": [P, P, I, P, I, I, I, I, I, P],
        "leb_attention_decode_prep_supported": [I, I, I, I, I, I],
        "leb_attention_decode_prep": [P, P, P, I, P, P, I, P, P, P, I, P, P, P, P, P, F, P, I, I, P, I, I, I, I, I, I, I, F, I, P],
        "leb_attention_prefill_supported": [I, I, I, I],
        "leb_attention_prefill_tc_supported": [I, I, I, I],
        "leb_attention_prefill_tc": [P, P, I, I, P, P, I, P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P],
        "leb_attention_pooled_tc": [P, P, I, I, P, P, I, P, I, P, P, I, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
        "leb_attention_pooled_tc_value_dim": [I],
        "leb_attention_prefill": [P, P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P],
        "leb_gemm_bf16_skinny_slices": [I, I],
        "leb_gemm_bf16_skinny_supported": [P, P, I, I, I],
        "leb_gemm_bf16_skinny": [P, I, P, P, I, I, I, I, I, I, P, I, P, I, I, F, P, P, P, P, P],
        "leb_gemm_bf16_skinny_conv": [P, P, P, I, I, I, I, I, P, P, P, P, P, I, P, I, P, I, I, F, P, P],
        "leb_gemm_bf16_tc_supported": [P, P, I, I],
        "leb_gemm_bf16_tc": [P, I, P, P, I, I, I, I, I, I, P, P],
        "leb_selftest_bounded_wait": [P, I, I, P],
        "leb_gemm_bf16_tc_slices": [I, I, I],
        "leb_gemm_bf16_tc_sliced": [P, I, P, P, I, I, I, I, I, I, P, I, P, P],
        "leb_gated_recurrence": [P, I, P, P, I, P, I, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, P],
        "leb_min_gru": [P, I, P, P, P, I, P, P, P, P, P, P, I, I, I, P, P],
        "leb_exp_gates": [P, P, P, P, P, I, P, P, F, P, P, P, P, I, I, I, P],
        "leb_exp_gates_finish": [P, I, P, P, P, I, P, F, F, I, I, I, P],
        "leb_layernorm_pair": [P, P, I, P, P, F, P, P, I, I, F, P],
        "leb_activation": [P, I, P, I, I, I, I, P],
        "leb_weighted_pair_sum": [P, P, P, F, P, F, I, I, I, P],
        "leb_attention_mixed": [P, P, P, I, P, P, I, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, P],
        "leb_attention_mixed_mma": [P, P, I, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P],
        "leb_attention_mixed_mma_supported": [I, I, I, I, I],
        "leb_delta_prep": [P, P, P, P, P, P, I, P, I, P, I, P, P, I, I, I, I, I, F, F, P],
        "leb_ssm_prep": [P, I, I, P, P, P, P, I, P, P, I, I, P],
        "leb_group_norm_gate": [P, I, P, P, I, P, I, I, I, I, F, I, P],
        "leb_postnorm_residual": [P, P, F, P, P, F, P, I, I, I, P],
        "leb_layernorm_bias": [P, I, P, P, P, P, I, I, F, P],
        "leb_embed_positions": [P, P, I, P, I, P, P, P, I, I, I, I, F, P],
        "leb_cast_rows": [P, I, P, S, P],
        "leb_pooled_attn_prep": [P, P, P, I, P, I, P, P, P, F, P, I, P, P, I, P, P, P, I, I, I, I, I, I, P],
        "leb_pool_blocks": [P, P, P, P, I, P, I, P, I, P, P, P, I, I, I, I, I, I, I, P],
        "leb_attention_pooled": [P, P, P, P, P, I, P, I, P, P, P, I, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P],
    }
    for name, args in sig.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = c_int
    L.leb_launch_count.restype = ctypes.c_longlong
    L.leb_launch_count.argtypes = []
    L.leb_sm_count.restype = c_int
    L.leb_sm_count.argtypes = []
    L.leb_set_latent_mma.restype = None
    L.leb_set_latent_mma.argtypes = [I]
    L.leb_retention_chunked_scratch.restype = ctypes.c_longlong
    L.leb_retention_chunked_scratch.argtypes = [I, I, I, I, I]
    for name, args in _OPTIONAL.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = c_int


# entry points that later files add; declared when present
_OPTIONAL: dict[str, list] = {}


class KernelError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().leb_last_error().decode())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (torch's raw accessor where it has one: a launch from Python
    costs some 25 us otherwise, most of it the Stream object)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _cuda(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}, the kernels run on CUDA only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")


def _dt(t: torch.Tensor, name: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{name}: unsupported dtype {t.dtype}") from None


# ----------------------------------------------------------------------------------------------
def embed(x: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0) -> None:
    """x[m] = table[tokens[m]] * scale as float."""
    _cuda(x, "embed.x", torch.float32)
    _cuda(table, "embed.table")
    _cuda(tokens, "embed.tokens", torch.int32)
    M, D = x.shape
    V = table.shape[0]
    assert table.shape[1] == D and tokens.numel() >= M
    _check(lib().leb_embed(_ptr(x), _ptr(table), _dt(table, "embed.table"), _ptr(tokens), M, D, V, float(scale), _stream()))


def rmsnorm(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float,
            rows: torch.Tensor | None = None, add: bool = False) -> None:
    """out = x * rsqrt(mean(x^2) + eps) * w  (out += ... when add).  x is float."""
    _cuda(out, "rmsnorm.out")
    _cuda(x, "rmsnorm.x", torch.float32)
    _cuda(w, "rmsnorm.w", torch.float32)
    M, D = out.shape
    assert x.shape[1] == D and w.numel() == D
    if rows is not None:
        _cuda(rows, "rmsnorm.rows", torch.int32)
        assert rows.numel() >= M
    else:
        assert x.shape[0] >= M
    _check(lib().leb_rmsnorm(_ptr(out), _dt(out, "rmsnorm.out"), _ptr(x), _ptr(w), _ptr(rows), M, D,
                             float(eps), 1 if add else 0, _stream()))


def layernorm(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
              bias: torch.Tensor | None = None) -> None:
    """out = (x - mean) / sqrt(var + eps) * w (+ bias) per row; x is float."""
    if bias is not None:
        _cuda(out, "layernorm.out")
        _cuda(x, "layernorm.x", torch.float32)
        _cuda(w, "layernorm.w", torch.float32)
        _cuda(bias, "layernorm.bias", torch.float32)
        M, D = out.shape
        assert x.shape[1] == D and w.numel() == D and bias.numel() == D
        if rows is not None:
            _cuda(rows, "layernorm.rows", torch.int32)
            assert rows.numel() >= M
        else:
            assert x.shape[0] >= M
        _check(lib().leb_layernorm_bias(_ptr(out), _dt(out, "layernorm.out"), _ptr(x), _ptr(w), _ptr(bias), _ptr(rows),
                                        M, D, float(eps), _stream()))
        return
    _cuda(out, "layernorm.out")
    _cuda(x, "layernorm.x", torch.float32)
    _cuda(w, "layernorm.w", torch.float32)
    M, D = out.shape
    assert x.shape[1] == D and w.numel() == D
    if rows is not None:
        _cuda(rows, "layernorm.rows", torch.int32)
        assert rows.numel() >= M
    else:
        assert x.shape[0] >= M
    _check(lib().leb_layernorm(_ptr(out), _dt(out, "layernorm.out"), _ptr(x), _ptr(w), _ptr(rows), M, D, float(eps), _stream()))


def scaled_residual(x: torch.Tensor, y: torch.Tensor, mult: float, h: torch.Tensor | None = None,
                    norm_w: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """x += mult * y (both float [M, D]); with `h` [M, D] the launch also leaves there the layer norm
    (weight `norm_w`, no bias) of the new rows."""
    _cuda(x, "scaled_residual.x", torch.float32)
    _cuda(y, "scaled_residual.y", torch.float32)
    M, D = x.shape
    assert y.shape == (M, D)
    if h is not None:
        _cuda(h, "scaled_residual.h")
        _cuda(norm_w, "scaled_residual.norm_w", torch.float32)
        assert h.shape == (M, D) and norm_w.numel() == D
    _check(lib().leb_scaled_residual(_ptr(x), _ptr(y), float(mult), _ptr(h), _dt(h, "scaled_residual.h") if h is not None else F32,
                                     _ptr(norm_w), float(eps), M, D, _stream()))


def postnorm_residual(x: torch.Tensor, y: torch.Tensor, alpha: float, w: torch.Tensor, bias: torch.Tensor | None,
                      eps: float, h: torch.Tensor | None = None) -> None:
    """x <- LN(alpha x + y) * w + bias per row (x, y float [M, D]); with `h` [M, D] the launch also leaves the
    new rows there in h's type (the input of the sublayer that reads the stream next)."""
    _cuda(x, "postnorm_residual.x", torch.float32)
    _cuda(y, "postnorm_residual.y", torch.float32)
    _cuda(w, "postnorm_residual.w", torch.float32)
    M, D = x.shape
    assert y.shape == (M, D) and w.numel() == D
    if bias is not None:
        _cuda(bias, "postnorm_residual.bias", torch.float32)
        assert bias.numel() == D
    if h is not None:
        _cuda(h, "postnorm_residual.h")
        assert h.shape == (M, D)
    _check(lib().leb_postnorm_residual(_ptr(x), _ptr(y), float(alpha), _ptr(w), _ptr(bias), float(eps), _ptr(h),
                                       _dt(h, "postnorm_residual.h") if h is not None else F32, M, D, _stream()))


def embed_positions(x: torch.Tensor, h: torch.Tensor | None, table: torch.Tensor, tokens: torch.Tensor,
                    positions: torch.Tensor, row_pos: torch.Tensor, scale: float = 1.0) -> None:
    """x[m] = table[tokens[m]] * scale + positions[row_pos[m]] as float; with `h`, the rows in h's type too."""
    _cuda(x, "embed_positions.x", torch.float32)
    _cuda(table, "embed_positions.table")
    _cuda(tokens, "embed_positions.tokens", torch.int32)
    _cuda(positions, "embed_positions.positions", torch.float32)
    _cuda(row_pos, "embed_positions.row_pos", torch.int32)
    M, D = x.shape
    assert table.shape[1] == D and positions.shape[1] == D and tokens.numel() >= M and row_pos.numel() >= M
    if h is not None:
        _cuda(h, "embed_positions.h")
        assert h.shape == (M, D)
    _check(lib().leb_embed_positions(_ptr(x), _ptr(h), _dt(h, "embed_positions.h") if h is not None else F32, _ptr(table),
                                     _dt(table, "embed_positions.table"), _ptr(tokens), _ptr(positions), _ptr(row_pos),
                                     M, D, table.shape[0], positions.shape[0], float(scale), _stream()))


def cast_rows(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = x in out's type (x float, both contiguous and of one shape)."""
    _cuda(out, "cast_rows.out")
    _cuda(x, "cast_rows.x", torch.float32)
    assert out.numel() == x.numel()
    _check(lib().leb_cast_rows(_ptr(out), _dt(out, "cast_rows.out"), _ptr(x), x.numel(), _stream()))


def _f32_rows(t: torch.Tensor, name: str, M: int, width: int) -> int:
    """Checks a float [M, width] tensor that may be a column slice; returns its row stride."""
    _cuda(t, name, torch.float32, contiguous=False)
    assert t.shape == (M, width) and (width == 0 or t.stride(1) == 1), f"{name}: {tuple(t.shape)}, expected {(M, width)}"
    return t.stride(0)


def delta_prep(qn: torch.Tensor, kn: torch.Tensor, vs: torch.Tensor, g: torch.Tensor, wr: torch.Tensor, qkv: torch.Tensor,
               a: torch.Tensor, b: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, H: int, Gk: int, d: int, e: int,
               unit_eps: float, q_scale: float) -> None:
    """Between the convolutions and the recurrence of a delta-rule mixer (all float): q and k = silu, then unit
    vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale; v = silu; write strength sigmoid(b);
    decay exp(-exp(A_log_h) softplus(a + dt_bias)) per head and key channel.  qkv [M, 2 Gk d + H e] holds the
    convolved q | k | v; a [M, H d] and b [M, H] may be column slices."""
    M = qn.shape[0]
    for t, n, w in ((qn, "qn", Gk * d), (kn, "kn", Gk * d), (vs, "vs", H * e), (g, "g", H * d), (wr, "wr", H)):
        _cuda(t, f"delta_prep.{n}", torch.float32)
        assert t.shape == (M, w)
    ldq = _f32_rows(qkv, "delta_prep.qkv", M, 2 * Gk * d + H * e)
    lda = _f32_rows(a, "delta_prep.a", M, H * d)
    ldb = _f32_rows(b, "delta_prep.b", M, H)
    _cuda(dt_bias, "delta_prep.dt_bias", torch.float32)
    _cuda(A_log, "delta_prep.A_log", torch.float32)
    assert dt_bias.numel() == H * d and A_log.numel() == H
    _check(lib().leb_delta_prep(_ptr(qn), _ptr(kn), _ptr(vs), _ptr(g), _ptr(wr), _ptr(qkv), ldq, _ptr(a), lda, _ptr(b), ldb,
                                _ptr(dt_bias), _ptr(A_log), M, H, Gk, d, e, float(unit_eps), float(q_scale), _stream()))


def ssm_prep(xbc: torch.Tensor, conv_bias: torch.Tensor | None, dt: torch.Tensor, decay: torch.Tensor, dt_raw: torch.Tensor,
             dt_bias: torch.Tensor, A_log: torch.Tensor) -> None:
    """Between the convolution and the recurrence of a state-space mixer (all float): xbc <- silu(xbc + conv_bias)
    in place; dt = softplus(dt_raw + dt_bias) and decay = exp(-exp(A_log_h) dt), both [M, H]."""
    M, C = xbc.shape
    H = dt.shape[1]
    ldx = _f32_rows(xbc, "ssm_prep.xbc", M, C)
    ldt = _f32_rows(dt_raw, "ssm_prep.dt_raw", M, H)
    for t, n in ((dt, "dt"), (decay, "decay")):
        _cuda(t, f"ssm_prep.{n}", torch.float32)
        assert t.shape == (M, H)
    for t, n, w in ((conv_bias, "conv_bias", C), (dt_bias, "dt_bias", H), (A_log, "A_log", H)):
        if t is not None:
            _cuda(t, f"ssm_prep.{n}", torch.float32)
            assert t.numel() == w
    _check(lib().leb_ssm_prep(_ptr(xbc), ldx, C, _ptr(conv_bias), _ptr(dt), _ptr(decay), _ptr(dt_raw), ldt, _ptr(dt_bias),
                              _ptr(A_log), M, H, _stream()))


RECURRENCE_MAX_ROWS = 256     # rows of a head's state the recurrence kernel takes


def gated_recurrence(out: torch.Tensor, k: torch.Tensor, q: torch.Tensor, v: torch.Tensor, write: torch.Tensor,
                     decay: torch.Tensor, state: torch.Tensor, batch, H: int, Gk: int, d: int, e: int,
                     delta: bool, skip: torch.Tensor | None = None, ones_columns: int = 0) -> None:
    """The linear recurrence of the step's rows with a state per sequence and head (all float):
        S <- diag(decay) S;  u = write * v (delta: write * (v - S^T k));  S <- S + k u^T;  o = S^T q (+ skip_h v)
    k, q [M, Gk*d] (one row stride), v [M, H*e], write [M, H], decay [M, H*d] (per key channel) or [M, H];
    head h reads key head h // (H // Gk); state [slots, H, e, d] (a column of S is contiguous); out [M, H*e].
    `ones_columns` n > 0: v has e - n columns per head and the state's last n columns are written with ones, so
    they hold the (decayed, weighted) sum of the keys and their read-out is that sum's product with q."""
    M = out.shape[0]
    ev = e - int(ones_columns)
    assert 0 <= ev <= e and not (delta and ones_columns)
    ldo = _f32_rows(out, "gated_recurrence.out", M, H * e)
    ldk = _f32_rows(k, "gated_recurrence.k", M, Gk * d)
    assert _f32_rows(q, "gated_recurrence.q", M, Gk * d) == ldk
    ldv = _f32_rows(v, "gated_recurrence.v", M, H * ev)
    ldw = _f32_rows(write, "gated_recurrence.write", M, H)
    row_decay = decay.shape[1] == H * d and not (d == 1 and decay.shape[1] == H and False)
    if decay.shape[1] != H * d:
        row_decay = False
    ldd = _f32_rows(decay, "gated_recurrence.decay", M, H * d if row_decay else H)
    _cuda(state, "gated_recurrence.state", torch.float32)
    assert state.shape[1:] == (H, e, d)
    if skip is not None:
        _cuda(skip, "gated_recurrence.skip", torch.float32)
        assert skip.numel() == H
    single = batch.max_qlen == 1 and M == batch.n_seqs
    _check(lib().leb_gated_recurrence(_ptr(out), ldo, _ptr(k), _ptr(q), ldk, _ptr(v), ldv, _ptr(write), ldw, _ptr(decay), ldd,
                                      1 if row_decay else 0, 1 if delta else 0, _ptr(skip), _ptr(state), _ptr(batch.seq_slot),
                                      _ptr(batch.seq_qstart), None if single else _ptr(batch.seq_qlen), batch.n_seqs,
                                      H, Gk, d, e, ev, _stream()))


def group_norm_gate(out: torch.Tensor, y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, group_size: int, eps: float,
                    gate_first: bool) -> None:
    """Groups of `group_size` neighbouring numbers of a row of y (float [M, C]) divided by their root mean square,
    times w[j % len(w)], gated by z (float [M, C], a column slice is fine): times sigmoid(z) after the norm, or
    (gate_first) y silu(z) before it.  out [M, C] in the activation type."""
    _cuda(out, "group_norm_gate.out")
    M, C = out.shape
    _cuda(y, "group_norm_gate.y", torch.float32)
    assert y.shape == (M, C)
    ldz = _f32_rows(z, "group_norm_gate.z", M, C)
    _cuda(w, "group_norm_gate.w", torch.float32)
    _check(lib().leb_group_norm_gate(_ptr(out), _dt(out, "group_norm_gate.out"), _ptr(y), _ptr(z), ldz, _ptr(w), M, C,
                                     int(group_size), w.numel(), float(eps), 1 if gate_first else 0, _stream()))


def min_gru(out: torch.Tensor, pz: torch.Tensor, px: torch.Tensor, pg: torch.Tensor, bz: torch.Tensor | None,
            bx: torch.Tensor | None, state: torch.Tensor, batch, scratch: torch.Tensor | None = None) -> None:
    """The minimal gated recurrent unit over the step's rows, per channel and sequence (all float):
    z = sigmoid(pz + bz), u = px + bx, c = u + 1/2 where u >= 0 else sigmoid(u), S <- (1 - z) S + z c,
    out = S * silu(pg) in out's type.  pz, px, pg float [M, W] with one row stride; state [slots, W].  `scratch`
    (float, `min_gru_scratch` numbers): sequences that bring many rows then run in pieces side by side."""
    _cuda(out, "min_gru.out")
    M, W = out.shape
    ldp = _f32_rows(pz, "min_gru.pz", M, W)
    assert _f32_rows(px, "min_gru.px", M, W) == ldp and _f32_rows(pg, "min_gru.pg", M, W) == ldp
    for name, t in (("bz", bz), ("bx", bx)):
        if t is not None:
            _cuda(t, f"min_gru.{name}", torch.float32)
            assert t.numel() == W
    _cuda(state, "min_gru.state", torch.float32)
    assert state.shape[1:] == (W,)
    single = batch.max_qlen == 1 and M == batch.n_seqs
    if scratch is not None:
        _cuda(scratch, "min_gru.scratch", torch.float32)
        if scratch.numel() < min_gru_scratch(batch, W):
            raise KernelError(f"min_gru: scratch of {scratch.numel()} numbers, {min_gru_scratch(batch, W)} needed")
    _check(lib().leb_min_gru(_ptr(out), _dt(out, "min_gru.out"), _ptr(pz), _ptr(px), _ptr(pg), ldp, _ptr(bz), _ptr(bx),
                             _ptr(state), _ptr(batch.seq_slot), _ptr(batch.seq_qstart),
                             None if single else _ptr(batch.seq_qlen), batch.n_seqs, W, batch.max_qlen, _ptr(scratch),
                             _stream()))


_gru_piece = [0]


def min_gru_scratch(batch, W: int) -> int:
    """Floats of scratch with which `min_gru` runs a step's long sequences in pieces (0: the step has none)."""
    if not _gru_piece[0]:
        fn = lib().leb_min_gru_piece_rows
        fn.restype, fn.argtypes = c_int, []
        _gru_piece[0] = int(fn())
    if batch.max_qlen <= _gru_piece[0]:
        return 0
    return 2 * batch.n_seqs * (-(-batch.max_qlen // _gru_piece[0])) * W


def exp_gates(decay: torch.Tensor, write: torch.Tensor, mrow: torch.Tensor, pi: torch.Tensor, pf: torch.Tensor,
              bi: torch.Tensor | None, bf: torch.Tensor | None, cap: float, mstate: torch.Tensor, batch) -> None:
    """Exponential gates under a running maximum, per head and sequence (all float): i = cap tanh((pi + bi) / cap),
    f = logsigmoid(cap tanh((pf + bf) / cap)), m_t = max(f_t + m_(t-1), i_t) from the carried m (mstate [slots, H]),
    decay_t = exp(f_t + m_(t-1) - m_t), write_t = exp(i_t - m_t), mrow_t = m_t.  All [M, H]."""
    _cuda(decay, "exp_gates.decay", torch.float32)
    M, H = decay.shape
    _cuda(write, "exp_gates.write", torch.float32)
    _cuda(mrow, "exp_gates.mrow", torch.float32)
    assert write.shape == (M, H) and mrow.shape == (M, H)
    ldp = _f32_rows(pi, "exp_gates.pi", M, H)
    assert _f32_rows(pf, "exp_gates.pf", M, H) == ldp
    for name, t in (("bi", bi), ("bf", bf)):
        if t is not None:
            _cuda(t, f"exp_gates.{name}", torch.float32)
            assert t.numel() == H
    _cuda(mstate, "exp_gates.mstate", torch.float32)
    assert mstate.shape[1:] == (H,)
    single = batch.max_qlen == 1 and M == batch.n_seqs
    _check(lib().leb_exp_gates(_ptr(decay), _ptr(write), _ptr(mrow), _ptr(pi), _ptr(pf), ldp, _ptr(bi), _ptr(bf), float(cap),
                               _ptr(mstate), _ptr(batch.seq_slot), _ptr(batch.seq_qstart),
                               None if single else _ptr(batch.seq_qlen), M, batch.n_seqs, H, _stream()))


def exp_gates_finish(out: torch.Tensor, y: torch.Tensor, mrow: torch.Tensor, gate: torch.Tensor, w: torch.Tensor,
                     qscale: float, eps: float, H: int, e: int) -> None:
    """The read-out of a memory with exponential gates on its way to the output projection: y float [M, H (e + 1)]
    holds per head the read-out and, in its last column, the normaliser's product with the query, both still
    without the query's scale; o = qscale y / (max(|qscale n.q|, exp(-m)) + 1e-6), divided by its root mean
    square per head, times w [H e], times sigmoid(gate) (float [M, H e], a column range is fine)."""
    _cuda(out, "exp_gates_finish.out")
    M = out.shape[0]
    assert out.shape == (M, H * e)
    _cuda(y, "exp_gates_finish.y", torch.float32)
    assert y.shape == (M, H * (e + 1))
    _cuda(mrow, "exp_gates_finish.mrow", torch.float32)
    assert mrow.shape == (M, H)
    ldg = _f32_rows(gate, "exp_gates_finish.gate", M, H * e)
    _cuda(w, "exp_gates_finish.w", torch.float32)
    assert w.numel() == H * e
    _check(lib().leb_exp_gates_finish(_ptr(out), _dt(out, "exp_gates_finish.out"), _ptr(y), _ptr(mrow), _ptr(gate), ldg,
                                      _ptr(w), float(qscale), float(eps), M, H, e, _stream()))


def layernorm_pair(h1: torch.Tensor, h2: torch.Tensor, x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float,
                   y: torch.Tensor | None = None, mult: float = 1.0) -> None:
    """Two layer norms (weights w1, w2, no bias) of the rows of x (float [M, D]) into h1 and h2; with `y` the
    launch first adds mult * y into x."""
    _cuda(x, "layernorm_pair.x", torch.float32)
    M, D = x.shape
    _cuda(h1, "layernorm_pair.h1")
    _cuda(h2, "layernorm_pair.h2", h1.dtype)
    assert h1.shape == (M, D) and h2.shape == (M, D)
    _cuda(w1, "layernorm_pair.w1", torch.float32)
    _cuda(w2, "layernorm_pair.w2", torch.float32)
    assert w1.numel() == D and w2.numel() == D
    if y is not None:
        _cuda(y, "layernorm_pair.y", torch.float32)
        assert y.shape == (M, D)
    _check(lib().leb_layernorm_pair(_ptr(h1), _ptr(h2), _dt(h1, "layernorm_pair.h1"), _ptr(x), _ptr(y), float(mult),
                                    _ptr(w1), _ptr(w2), M, D, float(eps), _stream()))


GELU_ERF, RELU_SQUARED = 0, 1      # activations without a gate (leb_activation); 2 and 3: the tanh form of gelu, silu
PLAIN_ACTIVATIONS = {"gelu": 0, "relu_squared": 1, "gelu_tanh": 2, "silu": 3}


PLAIN_ACT_BASE = 16      # a storing epilogue with an activation without a gate: STORE | (PLAIN_ACT_BASE + act) << 8


def plain_act_epilogue(act: int) -> int:
    """The epilogue code of a product that stores act(x . w^T); only for steps `stream_takes_plain_act` accepts."""
    return (PLAIN_ACT_BASE + int(act)) << 8


def stream_takes_plain_act(x: torch.Tensor, w: torch.Tensor, rows: int, n_groups: int = 0) -> bool:
    """Whether `linear` would run these rows through the weight stream of a decode step (dense: up to SMALL_M
    rows; grouped: up to 16 rows an expert), the products whose storing epilogue takes an activation without a
    gate.  Every other product leaves float results for `activation`."""
    if x.dtype != torch.bfloat16 or not w.is_contiguous():
        return False
    K = x.shape[1]
    if K % 8 != 0 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0 or w.data_ptr() % 16 != 0:
        return False
    if n_groups:
        return n_groups <= 256 and rows <= 16 * n_groups and (w.shape[1] * w.shape[2] * 2) % 16 == 0
    return rows <= SMALL_M


def activation(out: torch.Tensor, x: torch.Tensor, act: int) -> None:
    """out = act(x) in out's type; x float [M, F] (a column range is fine)."""
    _cuda(out, "activation.out")
    M, F_ = out.shape
    ldx = _f32_rows(x, "activation.x", M, F_)
    _check(lib().leb_activation(_ptr(out), _dt(out, "activation.out"), _ptr(x), ldx, M, F_, int(act), _stream()))


def weighted_pair_sum(out: torch.Tensor, y1: torch.Tensor, a: float, y2: torch.Tensor, b: float,
                      bias1: torch.Tensor | None = None, accumulate: bool = False) -> None:
    """out (+)= a (y1 + bias1) + b y2, all float [M, D]."""
    for n, t in (("out", out), ("y1", y1), ("y2", y2)):
        _cuda(t, f"weighted_pair_sum.{n}", torch.float32)
    M, D = out.shape
    assert y1.shape == (M, D) and y2.shape == (M, D)
    if bias1 is not None:
        _cuda(bias1, "weighted_pair_sum.bias1", torch.float32)
        assert bias1.numel() == D
    _check(lib().leb_weighted_pair_sum(_ptr(out), _ptr(y1), _ptr(bias1), float(a), _ptr(y2), float(b), M, D,
                                       1 if accumulate else 0, _stream()))


def add_row_vector(out: torch.Tensor, vec: torch.Tensor) -> None:
    """out[m, :] += vec (float)."""
    weighted_pair_sum(out, out, 1.0, out, 0.0, bias1=vec)


def mixed_attention_splits(batch, H: int, window: int) -> int:
    """In how many pieces a decode step's key range is cut: one block takes all heads of a row, so a step of few
    sequences would leave most SMs idle; pieces of at least 128 keys until the SMs have a block each."""
    if batch.max_qlen > 1:
        return 1
    keys = batch.max_kvlen if window <= 0 else min(batch.max_kvlen, window)
    return max(1, min(keys // 64, -(-2 * sm_count() // max(1, batch.n_seqs)), 32))


MIXED_MMA_MIN_ROWS = 8      # longest row count of a sequence from which bfloat16 prompts go to the tensor-core kernel
_MIXED_MMA = [True]


def set_mixed_attention_mma(on: bool) -> None:
    """Tests switch the tensor-core kernel of the mixed-heads attention off to compare it with the general one."""
    _MIXED_MMA[0] = bool(on)


def attention_mixed(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                    batch, talk: torch.Tensor, gate: torch.Tensor | None, nh: int, nkv: int, hd: int, vd: int,
                    page_size: int, window: int, scale: float, n_splits: int = 1, scratch: torch.Tensor | None = None) -> None:
    """Attention of the step's rows over the paged cache with the heads' scores mixed before the softmax:
    t_h = sum_g talk[h, g] (scale q_g . k), softmax over the visible keys (causal, inside `window` when > 0),
    weighted values, times sigmoid(gate) where a gate (float [M, nh vd], a column range is fine) is given."""
    _cuda(out, "attention_mixed.out")
    M = out.shape[0]
    _cuda(q, "attention_mixed.q", out.dtype, contiguous=False)
    assert out.shape == (M, nh * vd) and q.shape == (M, nh * hd) and q.stride(1) == 1
    _cuda(k_pool, "attention_mixed.k_pool", out.dtype)
    _cuda(v_pool, "attention_mixed.v_pool", out.dtype)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, vd, page_size)
    _cuda(block_table, "attention_mixed.block_table", torch.int32)
    _cuda(talk, "attention_mixed.talk", torch.float32)
    assert talk.shape == (nh, nh)
    ldg = _f32_rows(gate, "attention_mixed.gate", M, nh * vd) if gate is not None else 0
    if n_splits > 1:
        need = M * nh * n_splits * (vd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention_mixed: {n_splits} splits need {need} floats of scratch")
    single = batch.max_qlen == 1 and M == batch.n_seqs
    L = lib()
    if (_MIXED_MMA[0] and out.dtype == torch.bfloat16 and n_splits == 1 and batch.max_qlen >= MIXED_MMA_MIN_ROWS
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and L.leb_attention_mixed_mma_supported(nh, nkv, hd, vd, page_size)):
        _check(L.leb_attention_mixed_mma(
            _ptr(out), _ptr(q), q.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
            _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(talk), _ptr(gate),
            ldg, M, batch.n_seqs, nh, nkv, hd, vd, page_size, int(window), float(scale), batch.max_qlen, _stream()))
        return
    _check(lib().leb_attention_mixed(
        _ptr(out), _ptr(scratch), _ptr(q), q.stride(0), _ptr(k_pool), _ptr(v_pool), _dt(out, "attention_mixed"),
        _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
        None if single else _ptr(batch.seq_qlen), _ptr(talk), _ptr(gate), ldg, M, batch.n_seqs, nh, nkv, hd, vd, page_size,
        int(window), float(scale), batch.max_qlen, int(n_splits), _stream()))


def pooled_attn_prep(q_out: torch.Tensor, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, proj: torch.Tensor,
                     bias: torch.Tensor | None, q_norm_w: torch.Tensor | None, k_norm_w: torch.Tensor | None, eps: float,
                     freq_qk: torch.Tensor | None, rot: int, freq_v: torch.Tensor | None, block_table: torch.Tensor, batch,
                     nh: int, nkv: int, hd: int, vd: int, page_size: int) -> None:
    """The step's rows on their way into the windowed attention with rotated values: proj (float [M, (nh + nkv) hd +
    nkv vd], q | k | v) plus bias; q and k heads RMS-normed with a weight and rotated on their first `rot` numbers
    (split-half pairs, position * freq_qk); v heads rotated over their whole width (position * freq_v); q to q_out,
    k and v to the cache."""
    _cuda(q_out, "pooled_attn_prep.q_out")
    M = q_out.shape[0]
    assert q_out.shape == (M, nh * hd)
    ldp = _f32_rows(proj, "pooled_attn_prep.proj", M, (nh + nkv) * hd + nkv * vd)
    _cuda(k_pool, "pooled_attn_prep.k_pool", q_out.dtype)
    _cuda(v_pool, "pooled_attn_prep.v_pool", q_out.dtype)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, vd, page_size)
    _cuda(block_table, "pooled_attn_prep.block_table", torch.int32)
    for name, t, n in (("bias", bias, proj.shape[1]), ("q_norm_w", q_norm_w, hd), ("k_norm_w", k_norm_w, hd),
                       ("freq_qk", freq_qk, rot // 2), ("freq_v", freq_v, vd // 2)):
        if t is not None:
            _cuda(t, f"pooled_attn_prep.{name}", torch.float32)
            assert t.numel() == n, f"pooled_attn_prep.{name}: {t.numel()} numbers, expected {n}"
    _check(lib().leb_pooled_attn_prep(_ptr(q_out), _ptr(k_pool), _ptr(v_pool), _dt(q_out, "pooled_attn_prep"), _ptr(proj), ldp,
                                      _ptr(bias), _ptr(q_norm_w), _ptr(k_norm_w), float(eps), _ptr(freq_qk), int(rot) if freq_qk is not None else 0,
                                      _ptr(freq_v), _ptr(block_table), block_table.shape[1], _ptr(batch.row_seq),
                                      _ptr(batch.row_pos), _ptr(batch.seq_slot), M, nh, nkv, hd, vd, page_size, _stream()))


def pool_blocks(pk_pool: torch.Tensor, pv_pool: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                block_table: torch.Tensor, pool_table: torch.Tensor, batch, nkv: int, hd: int, vd: int, page_size: int,
                pool: int) -> None:
    """The pooled key and value (means over `pool` cached positions) of every block whose last position is among
    the step's rows, into the pooled pools at the block's number."""
    for t, n in ((pk_pool, "pk_pool"), (pv_pool, "pv_pool"), (v_pool, "v_pool")):
        _cuda(t, f"pool_blocks.{n}", k_pool.dtype)
    _cuda(k_pool, "pool_blocks.k_pool")
    assert pk_pool.shape[1:] == (nkv, page_size, hd) and pv_pool.shape[1:] == (nkv, vd, page_size)
    single = batch.max_qlen == 1 and batch.n_rows == batch.n_seqs
    _check(lib().leb_pool_blocks(_ptr(pk_pool), _ptr(pv_pool), _ptr(k_pool), _ptr(v_pool), _dt(k_pool, "pool_blocks"),
                                 _ptr(block_table), block_table.shape[1], _ptr(pool_table), pool_table.shape[1],
                                 _ptr(batch.seq_slot), _ptr(batch.seq_pos0), None if single else _ptr(batch.seq_qlen),
                                 batch.n_seqs, batch.max_qlen, nkv, hd, vd, page_size, int(pool), _stream()))


def pooled_attention_splits(batch, nkv: int, G: int, window: int, pool: int) -> int:
    """Blocks that share one sequence's key range in a decode step (1 for prompts): the range is the window plus
    the pooled blocks behind it; a split gets 128 keys or more, and no more blocks are made than run at once."""
    if batch.max_qlen != 1:
        return 1
    kv = max(int(batch.max_kvlen), 1)
    keys = min(kv, window) + (max(0, kv - window) // pool if pool > 0 else 0) if window > 0 else kv
    per = max(batch.n_seqs * nkv * ((G + 7) // 8), 1)
    return max(1, min(keys // 128, (4 * sm_count()) // per, 16))


def attention_pooled(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                     pk_pool: torch.Tensor | None, pv_pool: torch.Tensor | None, pool_table: torch.Tensor | None, batch,
                     head_scale: torch.Tensor, freq_v: torch.Tensor | None, nh: int, nkv: int, hd: int, vd: int,
                     page_size: int, window: int, pool: int, n_splits: int = 1, scratch: torch.Tensor | None = None) -> None:
    """Attention of the step's rows inside a window of `window` positions plus one pooled key and value for every
    block of `pool` positions wholly before the window (one softmax over both), scores times head_scale[h];
    the heads' results are turned back by their row's position (values are cached rotated) when freq_v is given."""
    _cuda(out, "attention_pooled.out")
    M = out.shape[0]
    _cuda(q, "attention_pooled.q", out.dtype)
    assert out.shape == (M, nh * vd) and q.shape == (M, nh * hd)
    _cuda(k_pool, "attention_pooled.k_pool", out.dtype)
    _cuda(v_pool, "attention_pooled.v_pool", out.dtype)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, vd, page_size)
    _cuda(block_table, "attention_pooled.block_table", torch.int32)
    pt_width = 0
    if pool > 0:
        _cuda(pk_pool, "attention_pooled.pk_pool", out.dtype)
        _cuda(pv_pool, "attention_pooled.pv_pool", out.dtype)
        _cuda(pool_table, "attention_pooled.pool_table", torch.int32)
        assert pk_pool.shape[1:] == (nkv, page_size, hd) and pv_pool.shape[1:] == (nkv, vd, page_size)
        pt_width = pool_table.shape[1]
    _cuda(head_scale, "attention_pooled.head_scale", torch.float32)
    assert head_scale.numel() == nh
    if freq_v is not None:
        _cuda(freq_v, "attention_pooled.freq_v", torch.float32)
        assert freq_v.numel() == vd // 2
    if n_splits > 1:
        need = M * nh * n_splits * (vd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention_pooled: {n_splits} splits need {need} floats of scratch")
    L = lib()
    if (out.dtype == torch.bfloat16 and n_splits == 1 and batch.max_qlen >= TC_ATTENTION_MIN_ROWS
            and q.stride(0) % 8 == 0 and L.leb_attention_prefill_tc_supported(nh, nkv, hd, page_size)
            and L.leb_attention_pooled_tc_value_dim(vd)):
        # prompts at the tensor-core kernel's sizes: pooled pages ahead of the window's, weights as two bfloat16 terms
        _check(L.leb_attention_pooled_tc(
            _ptr(out), _ptr(q), q.stride(0), M, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
            block_table.shape[1], _ptr(pk_pool) if pool > 0 else None, _ptr(pv_pool) if pool > 0 else None,
            pk_pool.shape[0] if pool > 0 else 0, _ptr(pool_table) if pool > 0 else None, pt_width, _ptr(batch.seq_slot),
            _ptr(batch.seq_pos0), _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(head_scale), _ptr(freq_v),
            batch.n_seqs, nh, nkv, hd, vd, page_size, int(window), int(pool), batch.max_qlen,
            _ptr(_status_word(out.device)), _stream()))
        return
    single = batch.max_qlen == 1 and M == batch.n_seqs
    _check(L.leb_attention_pooled(
        _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _dt(out, "attention_pooled"), _ptr(block_table),
        block_table.shape[1], _ptr(pk_pool) if pool > 0 else None, _ptr(pv_pool) if pool > 0 else None,
        _ptr(pool_table) if pool > 0 else None, pt_width, _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
        None if single else _ptr(batch.seq_qlen), _ptr(batch.row_pos), _ptr(head_scale), _ptr(freq_v), M, batch.n_seqs,
        nh, nkv, hd, vd, page_size, int(window), int(pool), batch.max_qlen, int(n_splits), _stream()))


def swiglu(out: torch.Tensor, gu: torch.Tensor) -> None:
    """out[m, j] = silu(gu[m, j]) * gu[m, F + j]."""
    _cuda(out, "swiglu.out")
    _cuda(gu, "swiglu.gu")
    M, Fd = out.shape
    assert gu.shape == (M, 2 * Fd)
    _check(lib().leb_swiglu(_ptr(out), _dt(out, "swiglu.out"), _ptr(gu), _dt(gu, "swiglu.gu"), M, Fd, _stream()))


SILU, GELU_TANH, CLAMPED_SIGMOID = 0, 1, 2      # activations of a gated feed-forward


def gated_act(out: torch.Tensor, gu: torch.Tensor, act: int, limit: float = 0.0, alpha: float = 1.0) -> None:
    """out[m, j] = act(gu[m, j]) * gu[m, F + j], act SILU or GELU_TANH; or CLAMPED_SIGMOID: with
    g = min(gu[m, j], limit) and u = clamp(gu[m, F + j], -limit, limit), g * sigmoid(alpha * g) * (u + 1)."""
    _cuda(out, "gated_act.out")
    _cuda(gu, "gated_act.gu")
    M, Fd = out.shape
    assert gu.shape == (M, 2 * Fd)
    _check(lib().leb_gated_act(_ptr(out), _dt(out, "gated_act.out"), _ptr(gu), _dt(gu, "gated_act.gu"), M, Fd,
                               int(act), float(limit), float(alpha), _stream()))


def gated_residual(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, bias: torch.Tensor | None,
                   h: torch.Tensor | None = None, norm_w: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """x += y * sigmoid(z + bias): x and y float [M, D], z the gate's pre-activation [M, D] (a column
    slice is fine), bias float [D].  With `h` [M, D] the launch also leaves there the RMS norm of the
    new rows with the weight `norm_w` (the input of whatever reads the stream next)."""
    _cuda(x, "gated_residual.x", torch.float32)
    _cuda(y, "gated_residual.y", torch.float32)
    _cuda(z, "gated_residual.z", contiguous=False)
    M, D = x.shape
    assert y.shape == (M, D) and z.shape == (M, D) and z.stride(1) == 1
    if bias is not None:
        _cuda(bias, "gated_residual.bias", torch.float32)
        assert bias.numel() == D
    if h is not None:
        _cuda(h, "gated_residual.h")
        _cuda(norm_w, "gated_residual.norm_w", torch.float32)
        assert h.shape == (M, D) and norm_w.numel() == D
    _check(lib().leb_gated_residual(_ptr(x), _ptr(y), _ptr(z), z.stride(0), _dt(z, "gated_residual.z"), _ptr(bias),
                                    _ptr(h), _dt(h, "gated_residual.h") if h is not None else F32, _ptr(norm_w),
                                    float(eps), M, D, _stream()))


def stream_add(x: torch.Tensor, x0: torch.Tensor | None, vec: torch.Tensor | None) -> None:
    """x[m] += x0[m] (if given) + vec (if given); all float."""
    _cuda(x, "stream_add.x", torch.float32)
    M, D = x.shape
    if x0 is not None:
        _cuda(x0, "stream_add.x0", torch.float32)
        assert x0.shape == (M, D)
    if vec is not None:
        _cuda(vec, "stream_add.vec", torch.float32)
        assert vec.numel() == D
    _check(lib().leb_stream_add(_ptr(x), _ptr(x0), _ptr(vec), M, D, _stream()))


def causal_conv(y: torch.Tensor, u: torch.Tensor, w: torch.Tensor, state: torch.Tensor, batch) -> None:
    """Causal depthwise convolution over time on every column of u [M, C] (a column slice is fine),
    taps [C, taps] float, with `state` [slots, C, taps-1] float holding each sequence's last
    projected values; writes y [M, C] and moves the state on."""
    _cuda(y, "causal_conv.y", contiguous=False)
    _cuda(u, "causal_conv.u", y.dtype, contiguous=False)
    _cuda(w, "causal_conv.w", torch.float32)
    M, C = y.shape
    taps = w.shape[1]
    assert u.shape == (M, C) and w.shape == (C, taps) and u.stride(1) == 1 and y.stride(1) == 1
    if taps > 1:
        _cuda(state, "causal_conv.state", torch.float32)
        assert state.shape[1:] == (C, taps - 1)
    else:
        state = None      # a single tap keeps nothing
    single = batch.max_qlen == 1 and M == batch.n_seqs
    _check(lib().leb_causal_conv(_ptr(y), y.stride(0), _ptr(u), u.stride(0), _dt(y, "causal_conv"), _ptr(w), _ptr(state),
                                 _ptr(batch.row_seq), _ptr(batch.seq_slot), _ptr(batch.seq_qstart), _ptr(batch.seq_qlen),
                                 M, batch.n_seqs, C, taps, 1 if single else 0, _stream()))


RETENTION_CHUNKED_MIN_ROWS = 16     # longest row count of a sequence from which a step runs the chunked form
_retention_ws: dict[int, list[torch.Tensor]] = {}


def _retention_workspace(device: torch.device, n_floats: int) -> torch.Tensor:
    """Float scratch for the chunk states; grows by adding buffers and never frees one (captured graphs)."""
    bufs = _retention_ws.setdefault(_device_index(device), [])
    if not bufs or bufs[-1].numel() < n_floats:
        bufs.append(torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device))
    return bufs[-1]


def retention(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
              state: torch.Tensor, decay: torch.Tensor, inv_freq: torch.Tensor | None, rot: int, k_scale: float,
              eps: float, batch, H: int, d: int, e: int) -> None:
    """Decayed linear attention of the step's rows with the per-sequence state [slots, H, d, e] (float):
    q and k rotated on their first `rot` dimensions, k scaled, S = decay S + k v^T, o = S^T q,
    o divided by its root mean square per head and multiplied by silu(g).  q, k [M, H*d] and v, g
    [M, H*e] are column slices of one projection."""
    _cuda(out, "retention.out")
    M = out.shape[0]
    assert out.shape == (M, H * e)
    ld = q.stride(0)
    for n, t, w in (("q", q, H * d), ("k", k, H * d), ("v", v, H * e), ("g", g, H * e)):
        _cuda(t, f"retention.{n}", out.dtype, contiguous=False)
        assert t.shape == (M, w) and t.stride(1) == 1 and t.stride(0) == ld
    _cuda(state, "retention.state", torch.float32)
    _cuda(decay, "retention.decay", torch.float32)
    assert state.shape[1:] == (H, d, e) and decay.numel() == H
    if rot:
        _cuda(inv_freq, "retention.inv_freq", torch.float32)
        assert inv_freq.numel() == rot // 2
    single = batch.max_qlen == 1 and M == batch.n_seqs
    L = lib()
    if batch.max_qlen >= RETENTION_CHUNKED_MIN_ROWS and L.leb_retention_chunked_supported(d, e):
        # many rows per sequence: chunks of the sequences side by side, the states between them by a scan
        scratch = _retention_workspace(out.device, int(L.leb_retention_chunked_scratch(M, batch.n_seqs, H, d, e)))
        _check(L.leb_retention_chunked(_ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(g), ld, _dt(out, "retention"),
                                       _ptr(state), _ptr(scratch), _ptr(decay), _ptr(inv_freq), int(rot), float(k_scale),
                                       float(eps), _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
                                       _ptr(batch.seq_qlen), M, batch.n_seqs, H, d, e, _stream()))
        return
    _check(L.leb_retention(_ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(g), ld, _dt(out, "retention"), _ptr(state),
                               _ptr(decay), _ptr(inv_freq), int(rot), float(k_scale), float(eps), _ptr(batch.seq_slot),
                               _ptr(batch.seq_pos0), _ptr(batch.seq_qstart), None if single else _ptr(batch.seq_qlen),
                               M, batch.n_seqs, H, d, e, _stream()))


def gather_rows(out: torch.Tensor, src: torch.Tensor, rows: torch.Tensor, div: int = 1) -> None:
    """out[p] = src[rows[p] // div]."""
    _cuda(out, "gather_rows.out")
    _cuda(src, "gather_rows.src", out.dtype)
    _cuda(rows, "gather_rows.rows", torch.int32)
    P_, D = out.shape
    assert src.shape[1] == D and rows.numel() >= P_
    _check(lib().leb_gather_rows(_ptr(out), _ptr(src), _dt(out, "gather_rows"), _ptr(rows), div, P_, D, _stream()))


def add_(x: torch.Tensor, y: torch.Tensor) -> None:
    _cuda(x, "add.x", torch.float32)
    _cuda(y, "add.y", torch.float32)
    assert x.numel() == y.numel()
    _check(lib().leb_add(_ptr(x), _ptr(y), x.numel(), _stream()))


def shortconv(y: torch.Tensor, bcx: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None,
              state: torch.Tensor, batch, Lc: int) -> None:
    """Gated short convolution over the step's rows; updates `state` [slots, D, Lc-1] (float)."""
    _cuda(y, "shortconv.y")
    _cuda(bcx, "shortconv.bcx", y.dtype)
    _cuda(w, "shortconv.w", torch.float32)
    _cuda(state, "shortconv.state", torch.float32)
    M, D = y.shape
    assert bcx.shape == (M, 3 * D) and w.numel() == D * Lc
    assert state.shape[1:] == (D, Lc - 1)
    if bias is not None:
        _cuda(bias, "shortconv.bias", torch.float32)
    single = batch.max_qlen == 1 and M == batch.n_seqs     # decode: the one-launch form
    _check(lib().leb_shortconv(_ptr(y), _ptr(bcx), _dt(y, "shortconv"), _ptr(w), _ptr(bias), _ptr(state),
                               _ptr(batch.row_seq), _ptr(batch.seq_slot), _ptr(batch.seq_qstart),
                               None if single else _ptr(batch.seq_qlen), M, batch.n_seqs, D, Lc, _stream()))


CONV_FUSED_MAX_LC = 5    # conv lengths the fused decode kernel takes


def shortconv_decode_fused(y: torch.Tensor, h: torch.Tensor, w_in: torch.Tensor, w: torch.Tensor,
                           bias: torch.Tensor | None, state: torch.Tensor, batch, Lc: int,
                           scale: "SplitNorm | None" = None) -> bool:
    """The conv mixer's in_proj and convolution of a decode step without a kernel of the
    convolution's own: y = conv(h . w_in^T), state updated.  Up to SMALL_M sequences it is the epilogue
    of the weight stream (one launch); up to SKINNY_M sequences the second kernel of the sliced
    tcgen05 product.  False (nothing done) when the step is not one of so many sequences with one
    bfloat16 row each, or the sizes are not the kernels'."""
    M, D = y.shape
    K = h.shape[1]
    if not (h.dtype == torch.bfloat16 and y.dtype == torch.bfloat16 and 0 < M <= SKINNY_M
            and batch.max_qlen == 1 and M == batch.n_seqs and 2 <= Lc <= CONV_FUSED_MAX_LC and K % 8 == 0
            and h.stride(0) % 8 == 0 and h.stride(1) == 1 and y.stride(1) == 1):
        return False
    if M > SMALL_M:
        L = lib()
        slices = L.leb_gemm_bf16_skinny_slices(3 * D, K)
        if slices < 2 or 3 * D >= SKINNY_MAX_N or not _tma_ok(h, w_in, K) or not w_in.is_contiguous():
            return False
        _cuda(w_in, "shortconv.w_in", torch.bfloat16)
        _cuda(w, "shortconv.w", torch.float32)
        _cuda(state, "shortconv.state", torch.float32)
        assert w_in.shape == (3 * D, K) and w.numel() == D * Lc and state.shape[1:] == (D, Lc - 1)
        if bias is not None:
            _cuda(bias, "shortconv.bias", torch.float32)
        ssq, parts, d_in, eps = _scale_args(scale, M, K)
        part = _skinny_workspace(h.device, slices * M * 3 * D)
        _check(L.leb_gemm_bf16_skinny_conv(_ptr(y), _ptr(h), _ptr(w_in), M, D, K, h.stride(0), y.stride(0), _ptr(w),
                                           _ptr(bias), _ptr(state), _ptr(batch.row_seq), _ptr(batch.seq_slot), Lc,
                                           _ptr(part), slices, ssq, parts, d_in, eps, _ptr(_status_word(h.device)),
                                           _stream()))
        return True
    _cuda(h, "shortconv.h", contiguous=False)
    _cuda(w_in, "shortconv.w_in", torch.bfloat16)
    _cuda(w, "shortconv.w", torch.float32)
    _cuda(state, "shortconv.state", torch.float32)
    assert w_in.shape == (3 * D, K) and w.numel() == D * Lc and state.shape[1:] == (D, Lc - 1)
    if bias is not None:
        _cuda(bias, "shortconv.bias", torch.float32)
    ssq, parts, d_in, eps = _scale_args(scale, M, K)
    _check(lib().leb_gemm_bf16_stream_conv(_ptr(y), _ptr(h), _ptr(w_in), M, D, K, h.stride(0), y.stride(0), _ptr(w),
                                           _ptr(bias), _ptr(state), _ptr(batch.row_seq), _ptr(batch.seq_slot), Lc,
                                           ssq, parts, d_in, eps, _stream()))
    return True


def qk_rope_store(q_out: torch.Tensor, q_in: torch.Tensor, k_in: torch.Tensor | None,
                  v_in: torch.Tensor | None, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
                  block_table: torch.Tensor, batch, q_norm_w, k_norm_w, eps: float,
                  inv_freq: torch.Tensor | None, rope_dim: int, neox: bool, nh: int, nkv: int, hd: int,
                  page_size: int, vd: int | None = None, v_norm: bool = False, hd_in: int | None = None,
                  vd_in: int | None = None) -> None:
    """Per-head norm and rotation of q and k; k and v go to the paged cache, q to q_out.

    q_in/k_in/v_in may be column slices of one fused projection (row stride = its width).
    `vd`: width of a value head where it is not the key head's; `v_norm`: every value head is
    divided by its root mean square (with `eps`, no weight) before it is stored.  `hd_in` / `vd_in`:
    width of a head in q_in/k_in and in v_in where heads are stored wider than they are (hd in q_out
    and the key pool, vd in the value pool; the rest of a stored head is zeros, the norms run over the
    head as it comes).
    """
    vd = hd if vd is None else int(vd)
    hd_in = hd if hd_in is None else int(hd_in)
    vd_in = vd if vd_in is None else int(vd_in)
    assert hd_in <= hd and vd_in <= vd and q_out.shape[1] == nh * hd
    _cuda(q_out, "qk_rope_store.q_out")
    _cuda(q_in, "qk_rope_store.q_in", q_out.dtype, contiguous=False)
    M = q_out.shape[0]
    assert q_in.stride(-1) == 1 and q_in.shape == (M, nh * hd_in)
    q_stride = q_in.stride(0)
    kv_stride = 0
    if k_in is not None:
        _cuda(k_in, "qk_rope_store.k_in", q_out.dtype, contiguous=False)
        _cuda(v_in, "qk_rope_store.v_in", q_out.dtype, contiguous=False)
        assert k_in.shape == (M, nkv * hd_in) and v_in.shape == (M, nkv * vd_in)
        assert k_in.stride(0) == v_in.stride(0) and k_in.stride(-1) == 1 and v_in.stride(-1) == 1
        kv_stride = k_in.stride(0)
        _cuda(k_pool, "qk_rope_store.k_pool", q_out.dtype)
        _cuda(v_pool, "qk_rope_store.v_pool", q_out.dtype)
        assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, vd, page_size)
    _cuda(block_table, "qk_rope_store.block_table", torch.int32)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("inv_freq", inv_freq)):
        if t is not None:
            _cuda(t, f"qk_rope_store.{name}", torch.float32)
    if inv_freq is not None:
        assert inv_freq.numel() == rope_dim // 2
    _check(lib().leb_qk_rope_store(
        _ptr(q_out), _ptr(q_in), q_stride, _ptr(k_in), _ptr(v_in), kv_stride, _ptr(k_pool), _ptr(v_pool),
        _dt(q_out, "qk_rope_store"), _ptr(block_table), block_table.shape[1], _ptr(batch.row_seq),
        _ptr(batch.row_pos), _ptr(batch.seq_slot), _ptr(q_norm_w), _ptr(k_norm_w), float(eps),
        _ptr(inv_freq), rope_dim, 1 if neox else 0, M, nh, nkv, hd, page_size, vd, 1 if v_norm else 0, hd_in, vd_in,
        _stream()))


_sm_counts: dict[int, int] = {}


def latent_prep(cq: torch.Tensor, proj: torch.Tensor, pool: torch.Tensor | None, block_table, batch,
                q_norm_w: torch.Tensor, kv_norm_w: torch.Tensor | None, eps: float, inv_freq: torch.Tensor | None,
                rot_dims: int, rank: int, rot: int, page_size: int) -> None:
    """The rows of a step of a latent-attention layer after the down projections: proj [M, q_rank
    (+ rank + rot)] -> cq [M, q_rank] = rmsnorm(proj[:, :q_rank]) * q_norm_w, and with `pool`
    [page, page_size, rank + rot] the cache row [rmsnorm(latent) * kv_norm_w | rotated key part] at every
    row's position (pairs (2i, 2i+1) of the first rot_dims dimensions turned by pos * inv_freq[i])."""
    _cuda(cq, "latent_prep.cq")
    _cuda(proj, "latent_prep.proj", cq.dtype, contiguous=False)
    _cuda(q_norm_w, "latent_prep.q_norm_w", torch.float32)
    M, q_rank = cq.shape
    assert proj.shape[0] == M and proj.stride(1) == 1 and q_norm_w.numel() == q_rank
    if pool is not None:
        _cuda(pool, "latent_prep.pool", cq.dtype)
        _cuda(kv_norm_w, "latent_prep.kv_norm_w", torch.float32)
        assert proj.shape[1] == q_rank + rank + rot and kv_norm_w.numel() == rank
        assert pool.shape[-1] == rank + rot and pool.shape[-2] == page_size
    if rot_dims:
        _cuda(inv_freq, "latent_prep.inv_freq", torch.float32)
        assert inv_freq.numel() == rot_dims // 2
    _check(lib().leb_latent_prep(_ptr(cq), _ptr(proj), proj.stride(0), _dt(cq, "latent_prep.cq"), _ptr(pool),
                                 _ptr(block_table), block_table.shape[1] if block_table is not None else 0,
                                 _ptr(batch.row_seq), _ptr(batch.row_pos), _ptr(batch.seq_slot), _ptr(q_norm_w),
                                 _ptr(kv_norm_w), float(eps), _ptr(inv_freq) if rot_dims else None, int(rot_dims), M, q_rank,
                                 int(rank), int(rot), int(page_size), _stream()))


def latent_q_split(qn: torch.Tensor, qr: torch.Tensor, q: torch.Tensor, row_pos: torch.Tensor,
                   inv_freq: torch.Tensor | None, rot_dims: int, H: int, dim: int, rot: int) -> None:
    """q [M, H * (dim + rot)] -> qn [H, M, dim_p] (each head's first `dim` numbers, head-major, zeros
    behind them) and qr [M, H, rot] (each head's last `rot` numbers, rotated by the row's position)."""
    _cuda(q, "latent_q_split.q")
    _cuda(qn, "latent_q_split.qn", q.dtype)
    _cuda(qr, "latent_q_split.qr", q.dtype)
    M = q.shape[0]
    dim_p = qn.shape[2]
    assert q.shape[1] == H * (dim + rot) and qn.shape[:2] == (H, M) and dim_p >= dim and qr.numel() == M * H * rot
    _check(lib().leb_latent_q_split(_ptr(qn), _ptr(qr), _ptr(q), _dt(q, "latent_q_split.q"), _ptr(row_pos),
                                    _ptr(inv_freq) if rot_dims else None, int(rot_dims), M, H, dim, dim_p, rot, _stream()))


def heads_to_rows(out: torch.Tensor, src: torch.Tensor) -> None:
    """src [H, M, w] -> out [M, H * w]."""
    _cuda(out, "heads_to_rows.out")
    _cuda(src, "heads_to_rows.src", out.dtype)
    H, M, w = src.shape
    assert out.shape == (M, H * w)
    _check(lib().leb_heads_to_rows(_ptr(out), _ptr(src), _dt(out, "heads_to_rows.out"), M, H, w, _stream()))


def latent_attention_uses_mma(dtype: torch.dtype, rank: int, rot: int, page_size: int, ld_out: int) -> bool:
    """Whether `latent_attention` runs its tensor-core kernel for these sizes (bfloat16, a latent that is a
    multiple of 32 up to 512, a rotated part that is a multiple of 16) or the general one."""
    return bool(_LATENT_MMA[0] and dtype == torch.bfloat16 and ld_out == rank
                and lib().leb_latent_attention_mma_supported(int(rank), int(rot), int(page_size)))


_LATENT_MMA = [True]


def set_latent_mma(on: bool) -> None:
    """Turns the tensor-core latent attention off (the general kernel then serves bfloat16 too) or on again."""
    _LATENT_MMA[0] = bool(on)
    lib().leb_set_latent_mma(1 if on else 0)


def latent_attention_splits(batch, H: int, mma: bool = False, rank: int = 0) -> int:
    """Pieces the key range of a decode step is cut into so that the blocks fill the SMs (1 for prompts).
    The tensor-core kernel takes up to 64 heads in a block that is alone on its SM, the general one 8 in
    blocks of which an SM holds several; a piece is at least 128 cached rows (measured at 2,048 positions:
    16 pieces of 128 rows are the fastest cut at batch 1 and 8 for latents of 256 and of 512)."""
    if batch.max_qlen != 1:
        return 1
    blocks = batch.n_seqs * -(-H // (64 if mma else 8))
    want = max(1, ((1 if mma else 2) * sm_count()) // max(1, blocks))
    return int(max(1, min(want, batch.max_kvlen // 128, 64)))


def latent_attention(out: torch.Tensor, qt: torch.Tensor, qr: torch.Tensor, pool: torch.Tensor, block_table, batch,
                     sink: torch.Tensor | None, rank: int, rot: int, page_size: int, scale: float,
                     n_splits: int = 1, scratch: torch.Tensor | None = None) -> None:
    """Causal attention of every row over its sequence's cached rows [c | k^r] (pool [page, page_size,
    rank + rot]): query vectors qt [H, M, rank] and qr [M, H, rot]; scores scale * ([qt | qr] . [c | k^r]);
    softmax with `sink` [H] as one more logit without a value; out [H, M, >= rank] = sum p c."""
    _cuda(out, "latent_attention.out")
    _cuda(qt, "latent_attention.qt", out.dtype)
    _cuda(qr, "latent_attention.qr", out.dtype)
    _cuda(pool, "latent_attention.pool", out.dtype)
    H, M, ld = out.shape
    assert qt.shape == (H, M, rank) and qr.numel() == M * H * rot and pool.shape[-1] == rank + rot and ld >= rank
    if sink is not None:
        _cuda(sink, "latent_attention.sink", torch.float32)
        assert sink.numel() == H
    if n_splits > 1:
        _cuda(scratch, "latent_attention.scratch", torch.float32)
        assert scratch.numel() >= M * H * n_splits * (rank + 2)
    _check(lib().leb_latent_attention(_ptr(out), ld, _ptr(scratch), _ptr(qt), _ptr(qr), _ptr(pool), _dt(out, "latent_attention.out"),
                                      _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
                                      _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(sink), M, batch.n_seqs, H, int(rank),
                                      int(rot), int(page_size), float(scale), batch.max_qlen, int(n_splits), _stream()))


def sm_count() -> int:
    """SMs of the current device, asked once per device."""
    d = torch.cuda.current_device()
    n = _sm_counts.get(d)
    if n is None:
        n = _sm_counts[d] = max(1, int(lib().leb_sm_count()))
    return n


def attention_splits(batch, nkv: int, G: int, sm_count: int | None = None, hd: int = 64) -> int:
    """How many blocks share one sequence's key range in a decode step (1 for prompts).

    Measured on B200 (head size 64, 8 kv heads, times with the merge of the splits): a block has a
    fixed cost of some microseconds, so a split must leave a block 256 positions or more (128 when
    there are so few blocks that the step waits on each one's latency); the blocks
    of a launch should all run at once (three per SM at head size 64: with 8 sequences of 4,096
    positions 6 splits, 384 blocks, take 14.7 us a layer and 7 splits, 448 blocks, 18.8 us); and
    when the sequences alone fill the GPU twice over, splitting pays only for long ranges (64
    sequences of 640 positions: 20.3 us unsplit, 27.4 us in 4 splits; of 4,096 positions: 110 us
    unsplit, 89 us in 4 splits).
    """
    if batch.max_qlen != 1:
        return 1
    if sm_count is None:
        sm_count = globals()["sm_count"]()
    kv = max(int(batch.max_kvlen), 1)
    per = max(batch.n_seqs * nkv * ((G + 15) // 16), 1)
    stage_bytes = 2 * 32 * hd * 2 * (3 if hd <= 32 else 2) * 4          # a block's rings: 4 warps, keys and values
    slots = sm_count * max(1, min(3, (227 * 1024) // stage_bytes))      # blocks that run at once
    if per >= 2 * sm_count:
        return 1 if kv < 2048 else min(4, kv // 1024)
    least = 128 if per * 8 <= sm_count else 256       # one or two sequences: latency counts, shorter blocks pay
    return max(1, min(slots // per, kv // least, 32))


TC_ATTENTION_MIN_ROWS = 8   # longest row count of a sequence from which prompts go to the tcgen05 attention


class RawQKV:
    """A decode step's q, k and v as the projection left them, for the decode attention kernel that
    norms, rotates and stores them itself (`decode_attention_takes_raw` says when it can)."""

    def __init__(self, q_in, k_in, v_in, q_norm_w, k_norm_w, eps, inv_freq, rope_dim, neox):
        self.q_in, self.k_in, self.v_in = q_in, k_in, v_in
        self.q_norm_w, self.k_norm_w, self.eps = q_norm_w, k_norm_w, float(eps)
        self.inv_freq, self.rope_dim, self.neox = inv_freq, int(rope_dim), bool(neox)


def decode_attention_takes_raw(dtype: torch.dtype, batch, M: int, nh: int, nkv: int, hd: int, page_size: int,
                               inv_freq, rope_dim: int, neox: bool) -> bool:
    """Whether `attention(..., raw=...)` will do the per-head norm, the rotation and the cache write
    of this step itself: a bfloat16 decode step (one row per sequence) whose sizes the tensor-core
    decode kernel takes, with a split-half rotation over the whole head."""
    return bool(dtype == torch.bfloat16 and batch.max_qlen == 1 and M == batch.n_seqs and inv_freq is not None
                and lib().leb_attention_decode_prep_supported(nh, nkv, hd, page_size, int(rope_dim), 1 if neox else 0))


def attention(out: torch.Tensor, q: torch.Tensor | None, k_pool: torch.Tensor, v_pool: torch.Tensor,
              block_table: torch.Tensor, batch, nh: int, nkv: int, hd: int, page_size: int,
              window: int, scale: float, gate: torch.Tensor | None = None,
              n_splits: int = 1, scratch: torch.Tensor | None = None, raw: RawQKV | None = None,
              vd: int | None = None) -> None:
    """Causal attention of the step's rows over the paged cache (which already holds their keys;
    with `raw`, the kernel puts the step's keys and values there itself and `q` is not used).
    `vd`: width of a value head where it differs from the key head's (the general kernel then)."""
    _cuda(out, "attention.out")
    if vd is not None and vd != hd:
        return _attention_general(out, q, k_pool, v_pool, block_table, batch, nh, nkv, hd, int(vd), page_size, window,
                                  scale, gate, n_splits, scratch)
    if raw is not None:
        return _attention_decode_raw(out, raw, k_pool, v_pool, block_table, batch, nh, nkv, hd, page_size, window,
                                     scale, gate, n_splits, scratch)
    _cuda(q, "attention.q", out.dtype)
    _cuda(k_pool, "attention.k_pool", out.dtype)
    _cuda(v_pool, "attention.v_pool", out.dtype)
    _cuda(block_table, "attention.block_table", torch.int32)
    M = out.shape[0]
    assert out.shape == (M, nh * hd) and q.shape == (M, nh * hd)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, hd, page_size)
    gate_stride = 0
    if gate is not None:
        _cuda(gate, "attention.gate", out.dtype, contiguous=False)
        assert gate.shape == (M, nh) and gate.stride(-1) == 1
        gate_stride = gate.stride(0)
    if n_splits > 1:
        need = M * nh * n_splits * (hd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention: {n_splits} splits need {need} floats of scratch")
        _cuda(scratch, "attention.scratch", torch.float32)
    L = lib()
    if (out.dtype == torch.bfloat16 and batch.max_qlen == 1 and M == batch.n_seqs
            and L.leb_attention_decode_supported(nh, nkv, hd, page_size)):
        # one row per sequence: the tensor-core decode kernel, then the merge of its splits
        _check(L.leb_attention_decode(
            _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
            block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
            _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale), n_splits,
            _stream()))
        if n_splits > 1:
            _check(L.leb_attention_merge(_ptr(out), _ptr(scratch), BF16, _ptr(gate), gate_stride, M, nh, hd,
                                         n_splits, _stream()))
        return
    if (out.dtype == torch.bfloat16 and n_splits == 1 and batch.max_qlen >= TC_ATTENTION_MIN_ROWS
            and q.stride(0) % 8 == 0 and L.leb_attention_prefill_tc_supported(nh, nkv, hd, page_size)):
        # prompts: tcgen05 tiles of 128 (position, head) rows, pages brought in by TMA
        _check(L.leb_attention_prefill_tc(
            _ptr(out), _ptr(q), q.stride(0), M, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
            block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart),
            _ptr(batch.seq_qlen), _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
            batch.max_qlen, _ptr(_status_word(out.device)), _stream()))
        return
    if (out.dtype == torch.bfloat16 and n_splits == 1
            and L.leb_attention_prefill_supported(nh, nkv, hd, page_size)):
        # rows of prompts (or decode without splits): the tensor-core kernel over (position, head) rows
        _check(L.leb_attention_prefill(
            _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
            _ptr(batch.seq_slot), _ptr(batch.seq_pos0), _ptr(batch.seq_qstart), _ptr(batch.seq_qlen),
            _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
            batch.max_qlen, _stream()))
        return
    _check(L.leb_attention(
        _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _dt(out, "attention"),
        _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
        _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(gate), gate_stride, M, batch.n_seqs, nh, nkv,
        hd, page_size, window, float(scale), batch.max_qlen, n_splits, hd, _stream()))


def _attention_general(out, q, k_pool, v_pool, block_table, batch, nh, nkv, hd, vd, page_size, window, scale, gate,
                       n_splits, scratch) -> None:
    """The general kernel with value heads of their own width."""
    _cuda(q, "attention.q", out.dtype)
    _cuda(k_pool, "attention.k_pool", out.dtype)
    _cuda(v_pool, "attention.v_pool", out.dtype)
    _cuda(block_table, "attention.block_table", torch.int32)
    M = out.shape[0]
    assert out.shape == (M, nh * vd) and q.shape == (M, nh * hd)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, vd, page_size)
    gate_stride = 0
    if gate is not None:
        _cuda(gate, "attention.gate", out.dtype, contiguous=False)
        assert gate.shape == (M, nh) and gate.stride(-1) == 1
        gate_stride = gate.stride(0)
    if n_splits > 1:
        need = M * nh * n_splits * (vd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention: {n_splits} splits need {need} floats of scratch")
    _check(lib().leb_attention(
        _ptr(out), _ptr(scratch), _ptr(q), _ptr(k_pool), _ptr(v_pool), _dt(out, "attention"),
        _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
        _ptr(batch.seq_qstart), _ptr(batch.seq_qlen), _ptr(gate), gate_stride, M, batch.n_seqs, nh, nkv,
        hd, page_size, window, float(scale), batch.max_qlen, n_splits, vd, _stream()))


def _attention_decode_raw(out, raw: RawQKV, k_pool, v_pool, block_table, batch, nh, nkv, hd, page_size, window,
                          scale, gate, n_splits, scratch) -> None:
    M = out.shape[0]
    if not decode_attention_takes_raw(out.dtype, batch, M, nh, nkv, hd, page_size, raw.inv_freq, raw.rope_dim, raw.neox):
        raise KernelError("attention: this step's q, k and v must be normed, rotated and stored before the call")
    _cuda(k_pool, "attention.k_pool", out.dtype)
    _cuda(v_pool, "attention.v_pool", out.dtype)
    _cuda(block_table, "attention.block_table", torch.int32)
    assert k_pool.shape[1:] == (nkv, page_size, hd) and v_pool.shape[1:] == (nkv, hd, page_size)
    _cuda(raw.q_in, "attention.q_in", out.dtype, contiguous=False)
    assert raw.q_in.shape == (M, nh * hd) and raw.q_in.stride(-1) == 1 and out.shape == (M, nh * hd)
    kv_stride = 0
    if raw.k_in is not None:
        _cuda(raw.k_in, "attention.k_in", out.dtype, contiguous=False)
        _cuda(raw.v_in, "attention.v_in", out.dtype, contiguous=False)
        assert raw.k_in.shape == (M, nkv * hd) and raw.v_in.shape == (M, nkv * hd)
        assert raw.k_in.stride(0) == raw.v_in.stride(0) and raw.k_in.stride(-1) == 1 and raw.v_in.stride(-1) == 1
        kv_stride = raw.k_in.stride(0)
    for name, t in (("q_norm_w", raw.q_norm_w), ("k_norm_w", raw.k_norm_w), ("inv_freq", raw.inv_freq)):
        if t is not None:
            _cuda(t, f"attention.{name}", torch.float32)
    assert raw.inv_freq.numel() == hd // 2
    gate_stride = 0
    if gate is not None:
        _cuda(gate, "attention.gate", out.dtype, contiguous=False)
        assert gate.shape == (M, nh) and gate.stride(-1) == 1
        gate_stride = gate.stride(0)
    if n_splits > 1:
        need = M * nh * n_splits * (hd + 2)
        if scratch is None or scratch.numel() < need or scratch.dtype != torch.float32:
            raise KernelError(f"attention: {n_splits} splits need {need} floats of scratch")
    L = lib()
    _check(L.leb_attention_decode_prep(
        _ptr(out), _ptr(scratch), _ptr(raw.q_in), raw.q_in.stride(0), _ptr(raw.k_in), _ptr(raw.v_in), kv_stride,
        _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(batch.seq_slot), _ptr(batch.seq_pos0),
        _ptr(batch.seq_qstart), _ptr(raw.q_norm_w), _ptr(raw.k_norm_w), raw.eps, _ptr(raw.inv_freq), raw.rope_dim,
        1 if raw.neox else 0, _ptr(gate), gate_stride, batch.n_seqs, nh, nkv, hd, page_size, window, float(scale),
        n_splits, _stream()))
    if n_splits > 1:
        _check(L.leb_attention_merge(_ptr(out), _ptr(scratch), BF16, _ptr(gate), gate_stride, M, nh, hd, n_splits, _stream()))


# ----------------------------------------------------------------------------------------------
STORE, ACCUMULATE, SWIGLU = 0, 1, 2
GEGLU = SWIGLU | (GELU_TANH << 8)     # the gated epilogue with the tanh form of gelu: the activation rides in the upper bits
CLAMPED_SIGMOID_SLOPE = 1.702     # the slope the fused form of the clamped activation is built with


def gated_epilogue(act: int, limit: float = 0.0, alpha: float = 1.0) -> int | None:
    """The epilogue code of a bfloat16 product that applies act(gate) * up itself, or None where the
    activation has no fused form (the clamped one with another slope, or a limit bfloat16 does not hold
    exactly: the limit travels in the code as the upper half of its float)."""
    if act in (SILU, GELU_TANH):
        return SWIGLU | (act << 8)
    if act == CLAMPED_SIGMOID and alpha == CLAMPED_SIGMOID_SLOPE and limit > 0:
        bits = int(torch.tensor(float(limit), dtype=torch.float32).view(torch.int32))
        if bits & 0xFFFF == 0:
            return SWIGLU | (CLAMPED_SIGMOID << 8) | ((bits >> 16) << 16)
    return None


SMALL_M = 16  # rows up to which the weight-streaming kernel is used; above, tcgen05 tiles


# Forming the norm inside a product (in the consumer's prologue, or in the tail of the product
# before it) was built and measured slower than the separate norm kernel each time: with
# programmatic dependent launch the small norm kernel between two products is the window in which
# the next product starts up and fetches its first weights.  So the norm stays a kernel of its own.


class SplitNorm:
    """An RMSNorm split between the product before it and the product after it (decode steps).

    `values` [M, D] is bfloat16(x * weight) and `ssq` [M, ceil(D/16)] holds partial sums of x^2,
    both left by the product that added into the residual x (`linear(..., emit=...)`); the product
    that takes `values` as its input multiplies its float sums by rsqrt(sum(ssq) / D + eps)
    (`linear(..., scale=...)`).  The products of steps of up to SKINNY_M rows do both (the weight
    stream up to SMALL_M rows, the sliced tcgen05 product above, in its second kernel);
    `split_norm_ok` says whether a step qualifies."""

    def __init__(self, values: torch.Tensor, ssq: torch.Tensor, weight: torch.Tensor, eps: float):
        self.values, self.ssq, self.weight, self.eps = values, ssq, weight, float(eps)
        self.filled = False      # set by the product that wrote values and ssq


def split_norm_ok(M: int, dtype: torch.dtype, reader_weight: torch.Tensor | None = None) -> bool:
    """Whether a step of M rows may split a norm in front of a product with `reader_weight`
    [N, K].  Once the norm is split its input exists only as bfloat16(x * g), so the product that
    reads it must be one that can scale its rows: the weight stream (up to SMALL_M rows) or the
    sliced tcgen05 product (up to SKINNY_M rows, N below its limit, operands TMA can fetch).  A
    reader that does not say what it multiplies with gets the split only where the weight stream
    runs."""
    if dtype != torch.bfloat16 or not 0 < M <= SKINNY_M:
        return False
    if reader_weight is None:
        return M <= SMALL_M
    if reader_weight.dim() != 2 or reader_weight.dtype != torch.bfloat16:
        return False
    N, K = reader_weight.shape
    if K % 8 != 0 or reader_weight.data_ptr() % 16 != 0:
        return False
    return M <= SMALL_M or N < SKINNY_MAX_N


def _scale_args(scale: "SplitNorm | None", M: int, K: int):
    if scale is None:
        return None, 0, 0, 0.0
    assert scale.filled and scale.values.shape == (M, K) and scale.ssq.shape[0] >= M
    return _ptr(scale.ssq), scale.ssq.shape[1], K, scale.eps


def linear(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE,
           group_offsets: torch.Tensor | None = None, rows_hint: int = 0, streaming: bool = False,
           scale: SplitNorm | None = None, emit: SplitNorm | None = None) -> None:
    """out (+)= x . w^T  with w [N, K] (or [E, N, K] with group_offsets [E+1] over the rows).

    float32 operands run on the CUDA cores in true 32-bit; bfloat16 operands on the tensor
    cores with float accumulation.  `epilogue`: STORE, ACCUMULATE (out is the float residual)
    or SWIGLU (w holds gate and up rows interleaved in blocks of 16; out has N/2 columns).
    Up to SMALL_M rows bfloat16 products stream W through shared memory with asynchronous copies;
    with more rows they go to the tcgen05 kernels: up to SKINNY_M rows with W as the wide operand
    and K cut into slices (a second kernel adds them up), above that 128 x BN tiles (K cut as well
    where a few hundred rows and a long K leave most SMs without a tile), from PAIRS_MIN_ROWS rows
    and large matrices 256 x 256 tiles on pairs of SMs; `streaming` asks for the register-fed
    weight-streaming kernel (the one that also serves grouped products) whatever the row count.
    """
    _cuda(x, "linear.x", contiguous=False)
    _cuda(w, "linear.w", x.dtype)
    _cuda(out, "linear.out", contiguous=False)
    M, K = x.shape
    assert x.stride(1) == 1 and out.stride(1) == 1
    lda, ldc = x.stride(0), out.stride(0)
    if group_offsets is not None:
        _cuda(group_offsets, "linear.group_offsets", torch.int32)
        E, N, Kw = w.shape
        assert group_offsets.numel() == E + 1
        stride = N * Kw
    else:
        N, Kw = w.shape
        E, stride = 1, 0
    assert Kw == K, f"linear: x has {K} columns, w has {Kw}"
    gated = (epilogue & 255) == SWIGLU
    n_out = N // 2 if gated else N
    assert out.shape == (M, n_out), f"linear: out is {tuple(out.shape)}, expected {(M, n_out)}"
    if M == 0:
        return
    L = lib()
    if x.dtype == torch.float32:
        if gated:
            raise KernelError("linear: the float path keeps the gated activation as its own kernel")
        if out.dtype != torch.float32:
            raise KernelError("linear: float operands need a float result")
        _check(L.leb_gemm_f32(_ptr(out), _ptr(x), _ptr(w), M, N, K, lda, ldc, epilogue, _ptr(group_offsets),
                              E, stride, _stream()))
        return
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported operand dtype {x.dtype}")
    if (K % 8 != 0 or lda % 8 != 0 or x.data_ptr() % 16 != 0 or w.data_ptr() % 16 != 0
            or (group_offsets is None and not w.is_contiguous())):
        # sizes the tensor-core kernels do not take (they fetch 16 bytes at a time): the plain product
        if gated or scale is not None or emit is not None:
            raise KernelError(f"linear: an inner size of {K} (row stride {lda}) takes neither a gated epilogue nor a split norm")
        if not w.is_contiguous():
            raise KernelError("linear: the weights of a grouped product must be contiguous")
        _check(L.leb_gemm_bf16_any(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc, epilogue,
                                   _ptr(group_offsets), E, stride, _stream()))
        return
    hint = rows_hint if rows_hint > 0 else M
    tc = _OPTIONAL_TC[0]
    ssq, parts, d_in, eps = _scale_args(scale, M, K)
    ev = eg = es = None
    if emit is not None and group_offsets is None and not streaming and M <= SKINNY_M:
        assert epilogue == ACCUMULATE and emit.values.shape == (M, N) and emit.ssq.shape == (M, -(-N // 16))
        assert emit.values.is_contiguous() and emit.ssq.is_contiguous() and emit.weight.numel() == N
        ev, eg, es = _ptr(emit.values), _ptr(emit.weight), _ptr(emit.ssq)
    if not streaming and group_offsets is None and M <= SMALL_M:
        # the decode step: W streamed through rings of asynchronous copies in shared memory
        _check(L.leb_gemm_bf16_stream(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                      epilogue, ssq, parts, d_in, eps, ev, eg, es, _stream()))
        if ev is not None:
            emit.filled = True
        return
    # few dozen rows: W as the wide operand with K sliced over blocks, unless N alone already gives
    # every SM several tiles (the output head), where the persistent kernel streams W better
    if (not streaming and group_offsets is None and SMALL_M < M <= SKINNY_M and N < SKINNY_MAX_N
            and linear_skinny(out, x, w, epilogue, norm_args=(ssq, parts, d_in, eps, ev, eg, es))):
        if ev is not None:
            emit.filled = True
        return
    if scale is not None:
        raise KernelError("linear: a split norm goes with the decode products of up to SKINNY_M rows only")
    if (not streaming and group_offsets is None and M >= PAIRS_MIN_ROWS and (N >= 4096 or K >= 4096)
            and linear_tc2(out, x, w, epilogue)):
        return      # many rows and a large weight matrix: 256 x 256 tiles on pairs of SMs
    if tc is not None and not streaming and group_offsets is None and M > SMALL_M and tc(out, x, w, epilogue):
        return
    if (not streaming and group_offsets is not None and E <= 256 and M > 16 * E and w.is_contiguous()
            and _tma_ok(x, w, K)):
        # experts with many rows each (prompts): tcgen05 tiles over the experts' row ranges
        _check(L.leb_gemm_bf16_tc_grouped(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                          epilogue, _ptr(group_offsets), E, _ptr(_status_word(x.device)), _stream()))
        return
    if not streaming and group_offsets is not None and E <= 256 and M <= 16 * E:
        # experts with a few rows each (decode steps): the ring-fed stream over the experts that have rows
        _check(L.leb_gemm_bf16_stream_grouped(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                              epilogue, _ptr(group_offsets), E, stride, _stream()))
        return
    _check(L.leb_gemm_bf16_small(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, lda, ldc,
                                 epilogue, _ptr(group_offsets), E, stride, hint, _stream()))


# set by ops.tc_gemm when the tensor-core (tcgen05) kernel is present
_OPTIONAL_TC: list = [None]


# ----------------------------------------------------------------------------------------------
def moe_router(topk_ids: torch.Tensor, topk_w: torch.Tensor, h: torch.Tensor, wr: torch.Tensor,
               bias: torch.Tensor | None, norm_topk: bool, scaling: float, softmax_chosen: bool = False,
               softmax_groups: tuple[int, int] | None = None, sigmoid_groups: tuple[int, int, int] | None = None) -> None:
    """The k experts of every row and their weights.  Default: sigmoid scores, the bias only chooses,
    weights are the chosen sigmoids (over their sum with norm_topk).  `softmax_chosen`: logits Wr h + bias,
    the k largest chosen, weights the softmax over the chosen logits alone.  `softmax_groups` = (groups, keep):
    scores are the softmax over all experts, the bias only chooses, only experts of the `keep` best of
    `groups` equal groups of neighbours (a group's score: its largest choice score) can be chosen, weights
    are the chosen scores over their sum (+ 1e-20).  `sigmoid_groups` = (groups, keep, top): sigmoid scores, the
    bias only chooses, groups as before with a group's score the sum of its `top` largest choice scores, weights
    the chosen scores over their sum (+ 1e-20) times `scaling`."""
    _cuda(topk_ids, "moe_router.topk_ids", torch.int32)
    _cuda(topk_w, "moe_router.topk_w", torch.float32)
    _cuda(h, "moe_router.h")
    _cuda(wr, "moe_router.wr", torch.float32)
    M, k = topk_ids.shape
    E, D = wr.shape
    assert h.shape == (M, D) and topk_w.shape == (M, k)
    if bias is not None:
        _cuda(bias, "moe_router.bias", torch.float32)
        assert bias.numel() == E
    mode = 2 if softmax_chosen else (1 if norm_topk else 0)
    if softmax_groups is not None:
        groups, keep = int(softmax_groups[0]), int(softmax_groups[1])
        if not (1 <= keep <= groups <= 255 and E % groups == 0 and keep * (E // groups) >= k):
            raise KernelError(f"moe_router: {keep} of {groups} groups over {E} experts cannot give {k} choices")
        mode = 3 | (groups << 8) | (keep << 16)
    if sigmoid_groups is not None:
        groups, keep, top = (int(v) for v in sigmoid_groups)
        if not (1 <= keep <= groups <= 255 and E % groups == 0 and keep * (E // groups) >= k and 1 <= top <= 15):
            raise KernelError(f"moe_router: {keep} of {groups} groups (ranked by their {top} best) over {E} experts "
                              f"cannot give {k} choices")
        mode = 4 | (groups << 8) | (keep << 16) | (top << 24)
    _check(lib().leb_moe_router(_ptr(topk_ids), _ptr(topk_w), _ptr(h), _dt(h, "moe_router.h"), _ptr(wr),
                                _ptr(bias), M, D, E, k, mode, float(scaling), _stream()))


def moe_align(offsets: torch.Tensor, sorted_pair: torch.Tensor, pair_row: torch.Tensor,
              topk_ids: torch.Tensor, E: int) -> None:
    for n, t in (("offsets", offsets), ("sorted_pair", sorted_pair), ("pair_row", pair_row),
                 ("topk_ids", topk_ids)):
        _cuda(t, f"moe_align.{n}", torch.int32)
    P_ = topk_ids.numel()
    assert offsets.numel() >= E + 1 and sorted_pair.numel() >= P_ and pair_row.numel() >= P_
    _check(lib().leb_moe_align(_ptr(offsets), _ptr(sorted_pair), _ptr(pair_row), _ptr(topk_ids), P_, E, _stream()))


def moe_combine(x: torch.Tensor, ys: torch.Tensor, pair_row: torch.Tensor, topk_w: torch.Tensor,
                accumulate: bool) -> None:
    _cuda(x, "moe_combine.x", torch.float32)
    _cuda(ys, "moe_combine.ys", torch.float32)
    _cuda(pair_row, "moe_combine.pair_row", torch.int32)
    _cuda(topk_w, "moe_combine.topk_w", torch.float32)
    M, D = x.shape
    k = topk_w.shape[1]
    assert ys.shape[1] == D and ys.shape[0] >= M * k and topk_w.shape[0] == M
    _check(lib().leb_moe_combine(_ptr(x), _ptr(ys), _ptr(pair_row), _ptr(topk_w), M, D, k,
                                 1 if accumulate else 0, _stream()))


# ----------------------------------------------------------------------------------------------
def penalties(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor,
              repeat_penalty: float, presence_penalty: float) -> None:
    _cuda(logits, "penalties.logits", torch.float32)
    _cuda(hist, "penalties.hist", torch.int32)
    _cuda(hist_len, "penalties.hist_len", torch.int32)
    n, V = logits.shape
    assert hist.shape[0] >= n
    _check(lib().leb_penalties(_ptr(logits), _ptr(hist), _ptr(hist_len), hist.shape[1], n, V,
                               float(repeat_penalty), float(presence_penalty), _stream()))


def penalties_slots(logits: torch.Tensor, hist: torch.Tensor, hist_len: torch.Tensor, seq_slot: torch.Tensor,
                    repeat_penalty: float, presence_penalty: float) -> None:
    """Penalises, in place, the tokens in each sequence's ring of recent tokens (hist [slots, window])."""
    _cuda(logits, "penalties_slots.logits", torch.float32)
    _cuda(hist, "penalties_slots.hist", torch.int32)
    _cuda(hist_len, "penalties_slots.hist_len", torch.int32)
    _cuda(seq_slot, "penalties_slots.seq_slot", torch.int32)
    n, V = logits.shape
    assert seq_slot.numel() >= n and hist_len.numel() == hist.shape[0]
    _check(lib().leb_penalties_slots(_ptr(logits), _ptr(hist), _ptr(hist_len), _ptr(seq_slot), hist.shape[1], n, V,
                                     float(repeat_penalty), float(presence_penalty), _stream()))


def history_append(hist: torch.Tensor, hist_len: torch.Tensor, seq_slot: torch.Tensor, chosen: torch.Tensor, n: int) -> None:
    """The chosen token of each of the first n sequences goes into its slot's ring."""
    _cuda(hist, "history_append.hist", torch.int32)
    _cuda(hist_len, "history_append.hist_len", torch.int32)
    _cuda(chosen, "history_append.chosen", torch.int32)
    assert seq_slot.numel() >= n and chosen.numel() >= n
    _check(lib().leb_history_append(_ptr(hist), _ptr(hist_len), _ptr(seq_slot), _ptr(chosen), hist.shape[1], n, _stream()))


def argmax(out: torch.Tensor, logits: torch.Tensor) -> None:
    _cuda(out, "argmax.out", torch.int32)
    _cuda(logits, "argmax.logits", torch.float32)
    n, V = logits.shape
    assert out.numel() >= n
    _check(lib().leb_argmax(_ptr(out), _ptr(logits), n, V, _stream()))


def sample(out: torch.Tensor, logits: torch.Tensor, u01: torch.Tensor, top_k: int, temperature: float,
           top_p: float, min_p: float) -> None:
    _cuda(out, "sample.out", torch.int32)
    _cuda(logits, "sample.logits", torch.float32)
    _cuda(u01, "sample.u01", torch.float32)
    n, V = logits.shape
    assert out.numel() >= n and u01.numel() >= n
    _check(lib().leb_sample(_ptr(out), _ptr(logits), _ptr(u01), n, V, int(top_k), float(temperature),
                            float(top_p), float(min_p), _stream()))


def advance(batch, chosen: torch.Tensor) -> None:
    """The chosen tokens become the step's input and every live sequence moves one position on."""
    _cuda(chosen, "advance.chosen", torch.int32)
    _check(lib().leb_advance(_ptr(batch.tokens), _ptr(batch.row_pos), _ptr(batch.seq_pos0), _ptr(batch.seq_slot),
                             _ptr(chosen), batch.n_seqs, _stream()))


def feed_tokens(batch, chosen: torch.Tensor) -> None:
    """Sequences with batch.feed[b] >= 0 take as their token what `chosen` holds at that place."""
    _cuda(chosen, "feed_tokens.chosen", torch.int32)
    _check(lib().leb_feed_tokens(_ptr(batch.tokens), _ptr(chosen), _ptr(batch.feed), batch.n_seqs, _stream()))


def launch_count() -> int:
    """Kernels this library has launched in this process (launches inside a replayed graph are
    counted once, when the graph was captured)."""
    return int(lib().leb_launch_count())


# ---- the tcgen05 matrix product ----------------------------------------------------------------
# The status word of a device sits right in front of the buffer the chosen tokens of a step go
# to, so that the copy that brings the tokens to the host brings the word along.
RESULT_TOKENS = 8192      # chosen tokens the shared buffer holds; larger steps use a buffer of their own
_STATUS_AT = 3            # the tokens then start on a 16-byte boundary
_tc_block: dict[int, torch.Tensor] = {}
_tc_status: dict[int, torch.Tensor] = {}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _status_block(device: torch.device) -> torch.Tensor:
    i = _device_index(device)
    if i not in _tc_block:
        _tc_block[i] = torch.zeros(_STATUS_AT + 1 + RESULT_TOKENS, dtype=torch.int32, device=device)
        _tc_status[i] = _tc_block[i][_STATUS_AT:_STATUS_AT + 1]
    return _tc_block[i]


def _status_word(device: torch.device) -> torch.Tensor:
    _status_block(device)
    return _tc_status[_device_index(device)]


def result_tokens(device: torch.device) -> torch.Tensor:
    """int32 [RESULT_TOKENS] for a step's chosen tokens, directly behind the device's status word."""
    return _status_block(device)[_STATUS_AT + 1:]


def status_and_tokens(device: torch.device, n: int) -> torch.Tensor:
    """The status word followed by the first n chosen tokens: what one copy brings to the host."""
    return _status_block(device)[_STATUS_AT:_STATUS_AT + 1 + n]


def raise_on_status(value: int, device: torch.device) -> None:
    """`value`: the status word as the host read it.  Non-zero: a kernel gave up on a bounded wait
    and what the step computed is not valid; the word is cleared and KernelError raised."""
    if value != 0:
        _status_word(device).zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting (role {value}) on cuda:{_device_index(device)}; "
                          "the step's result is not valid")


def check_device_status() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for i, t in _tc_status.items():
        raise_on_status(int(t.item()), t.device)


def selftest_bounded_wait(device: torch.device, limit: int = 2000, role: int = 9) -> None:
    """Launches one block that waits, with the kernels' own bounded wait, on a barrier nobody
    arrives on; it gives up after `limit` polls and sets the device's status word to `role`."""
    _check(lib().leb_selftest_bounded_wait(_ptr(_status_word(device)), int(limit), int(role), _stream()))


def _tma_ok(x: torch.Tensor, w: torch.Tensor, K: int) -> bool:
    """What leb_gemm_bf16_tc_supported checks (16-byte aligned bases and row strides), without the call."""
    return K > 0 and K % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def linear_tc(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE) -> bool:
    """out (+)= x . w^T on tcgen05 with TMA-fed tiles; False when the operands cannot go through TMA."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not _tma_ok(x, w, K):
        return False
    slices = L.leb_gemm_bf16_tc_slices(M, N, K) if N % 4 == 0 else 1
    if slices > 1:      # a few hundred rows and a long K: fewer tiles than SMs, so K is cut as well
        part = _skinny_workspace(x.device, slices * M * N)
        _check(L.leb_gemm_bf16_tc_sliced(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                         out.stride(0), epilogue, _ptr(part), slices,
                                         _ptr(_status_word(x.device)), _stream()))
        return True
    _check(L.leb_gemm_bf16_tc(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                              out.stride(0), epilogue, _ptr(_status_word(x.device)), _stream()))
    return True


PAIRS_MIN_ROWS = 1024   # rows from which the paired kernel is used (measured: 3-9% faster there, slower on small products)


def linear_tc2(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE) -> bool:
    """out (+)= x . w^T on pairs of SMs (tcgen05 cta_group::2, 256 x 256 tiles); False when the operands cannot go through TMA."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not _tma_ok(x, w, K):
        return False
    _check(L.leb_gemm_bf16_tc2(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                               out.stride(0), epilogue, _ptr(_status_word(x.device)), _stream()))
    return True


SKINNY_M = 128   # rows up to which W is the wide tcgen05 operand and K is sliced over blocks
SKINNY_MAX_N = 128 * 296   # from here on N alone gives every SM several tiles and the persistent kernel streams W better
_skinny_ws: dict[int, list[torch.Tensor]] = {}


def _skinny_workspace(device: torch.device, n_floats: int) -> torch.Tensor:
    """Float scratch for the K slices.  Grows by adding buffers and never frees one, so that a
    captured graph that points at an older buffer stays valid."""
    i = device.index if device.index is not None else torch.cuda.current_device()
    bufs = _skinny_ws.setdefault(i, [])
    if not bufs or bufs[-1].numel() < n_floats:
        bufs.append(torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device))
    return bufs[-1]


def linear_skinny(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int = STORE,
                  norm_args: tuple | None = None) -> bool:
    """out (+)= x . w^T for 1..128 rows with W as the wide tcgen05 operand and K sliced over blocks.
    `norm_args`: the halves of a split norm as `linear` unpacks them (its second kernel applies them)."""
    L = lib()
    M, K = x.shape
    N = w.shape[0]
    if not (1 <= M <= SKINNY_M and _tma_ok(x, w, K)):
        return False
    slices = L.leb_gemm_bf16_skinny_slices(N, K)
    ssq, parts, d_in, eps, ev, eg, es = norm_args or (None, 0, 0, 0.0, None, None, None)
    part = _skinny_workspace(x.device, slices * M * N) if slices > 1 else None
    _check(L.leb_gemm_bf16_skinny(_ptr(out), _dt(out, "linear.out"), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                  out.stride(0), epilogue, _ptr(part), slices, ssq, parts, d_in, eps, ev, eg, es,
                                  _ptr(_status_word(x.device)), _stream()))
    return True


_OPTIONAL_TC[0] = linear_tc
