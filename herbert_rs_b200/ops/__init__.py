"""Python faces of the kernels: one function per launcher of the kernel library.

Each function takes CUDA tensors, checks what only the host can check cheaply (device,
dtype, contiguity of the innermost axis) and launches on the current CUDA stream.  A launcher
that refuses its input raises `BackendError` with the launcher's own message.  Nothing here
computes on the CPU and nothing falls back to a library model or attention routine.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from ..errors import BackendError
from . import lib as _libmod
from .options import KernelOptions

F32, BF16 = 0, 1
ACT_SILU, ACT_GELU_TANH, ACT_GELU, ACT_RELU, ACT_SWISH_CLAMP = 0, 1, 2, 3, 4
# "swish_clamp" is a gated expert's: min(gate, L) sigmoid(1.702 min(gate, L)) (clamp(up, -L, L) + 1) with a limit L
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "gelu": ACT_GELU, "relu": ACT_RELU, "swish_clamp": ACT_SWISH_CLAMP}
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_ROWS = 64
# The one place where a choice between kernels can be changed (by a measurement script or a test
# that assigns its fields); nothing reads the environment.
options = KernelOptions()

_SIGS = {
    "hb_embed": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_void_p],
    "hb_scaled_residual_norm": [c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "hb_qk_prepare_cache": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p,
                            c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_rmsnorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "hb_swiglu": [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_add_residual": [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_qk_norm_rope_cache": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                              c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_simt": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_skinny_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gemm_skinny_norm_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                 c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "hb_finish_norm": [c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_gemm_tcgen05_norm_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_int, c_float, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p],
    "hb_gemm_tcgen05_norm_parts": [c_int, c_int],
    "hb_gemm_tcgen05_qkv_ok": [c_int, c_int],
    "hb_gemm_tcgen05_qkv_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
    "hb_gemm_tcgen05_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "hb_gemm_stream_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                            ctypes.c_longlong, c_void_p, c_int, c_void_p, c_void_p],
    "hb_attention_simt": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p,
                          c_int, c_void_p],
    "hb_attention_decode_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p],
    "hb_attention_decode_fused_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                       c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_attention_prefill_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p],
    "hb_attention_prefill_tc_bf16": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p,
                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "hb_argmax": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p],
    "hb_gemm_skinny_norm_parts": [c_int, c_int],
    "hb_sample": [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p],
    "hb_rng_normal": [c_int, c_void_p, ctypes.c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p],
    "hb_fill": [c_int, c_void_p, ctypes.c_longlong, c_float, c_void_p],
    "hb_cast": [c_int, c_void_p, c_int, c_void_p, ctypes.c_longlong, c_int, c_void_p],
    "hb_layernorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "hb_layernorm_residual": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "hb_latent_kv_store": [c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "hb_rotate_heads": [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int,
                        c_int, c_int, c_float, c_void_p],
    "hb_headwise_gemm": [c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                         c_int, c_int, c_int, c_float, c_void_p],
    "hb_latent_attention": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_moe_experts_grouped_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_moe_experts_tc_rows": [c_int, c_int, c_int],
    "hb_moe_experts_tc_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "hb_latent_attention_mma_ok": [c_int, c_int],
    "hb_latent_attention_mma_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "hb_gla_decay": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "hb_gla_scan": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_int, c_int, c_int, c_float, c_void_p],
    "hb_gla_output": [c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                      c_void_p],
    "hb_moe_route": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, c_float, c_void_p],
    "hb_moe_experts": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                       c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "hb_group_rmsnorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "hb_group_rmsnorm_residual": [c_int, c_void_p, c_int, c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_float, c_void_p],
    "hb_axpby": [c_void_p, c_int, c_float, c_void_p, c_int, c_float, c_int, c_int, c_void_p],
    "hb_bias_glu": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_tanh_cap": [c_void_p, c_int, c_float, c_int, c_int, c_void_p],
    "hb_short_conv": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_void_p],
    "hb_pair_embed": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_int, c_int, ctypes.c_longlong, ctypes.c_longlong, c_float, c_void_p],
    "hb_silu_columns": [c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "hb_delta_prepare": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p,
                         c_void_p, c_void_p, c_int, c_int, c_void_p],
    "hb_linear_scan": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_gated_rmsnorm": [c_int, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_void_p],
    "hb_qkv_rotary_cache": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_int, c_void_p],
    "hb_rotate_heads_back": [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_void_p],
    "hb_head_gate": [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "hb_general_delta_prepare": [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float,
                                 c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "hb_general_delta_scan": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                              c_int, c_void_p],
    "hb_gated_norm_residual": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                               c_float, c_void_p, c_int, c_int, c_void_p],
    "hb_token_gate": [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
}
_fns: dict = {}


def _fn(name: str):
    f = _fns.get(name)
    if f is None:
        lib = _libmod.load()
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise BackendError(f"kernel library has no entry point {name}") from None
        f.argtypes = _SIGS[name]
        f.restype = c_int
        _fns[name] = f
    return f


# kernels each launcher starts (for honest launch counts)
_KERNELS_PER_CALL = {"hb_attention_decode_bf16": 2, "hb_argmax": 2, "hb_sample": 2, "hb_moe_experts": 2,
                     "hb_moe_experts_grouped_bf16": 4, "hb_moe_experts_tc_bf16": 5}
_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (launches recorded into a graph count once)."""
    return _launches


_timeline = None     # while a `timed()` block is open: [(launcher name, start event, end event)]


def _run(name: str, *args) -> None:
    global _launches
    _launches += _KERNELS_PER_CALL.get(name, 1)
    if _timeline is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = _fn(name)(*args)
        e1.record()
        _timeline.append((name, e0, e1))
    else:
        rc = _fn(name)(*args)
    if rc != 0:
        raise BackendError(f"{name}: {_libmod.last_error()}")


class timed:
    """Where a step's time goes, by launcher: CUDA events around every launch made inside the block
    (eager steps only: a replayed graph makes no launches here).  The reference returns per-layer
    times on request in the same spirit (crates/core/src/backend.rs:97-102, profiler.rs:17-60).

        with ops.timed() as t:
            engine.step(...)
        t.by_kernel()     # {launcher: (launches, milliseconds)}, and "(between launches)"
    """

    def __enter__(self):
        global _timeline
        self._saved, _timeline = _timeline, []
        self._rows = _timeline
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = self._saved
        torch.cuda.synchronize()
        return False

    def by_kernel(self) -> dict:
        out: dict = {}
        for name, e0, e1 in self._rows:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + e0.elapsed_time(e1))
        if self._rows:
            whole = self._rows[0][1].elapsed_time(self._rows[-1][2])
            out["(between launches)"] = (len(self._rows) - 1, whole - sum(ms for _, ms in out.values()))
        return out


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current CUDA stream's handle (also the capturing stream while a graph is recorded).  Asked
    of torch's C layer directly where that entry exists: a step makes some two hundred launches, and
    `torch.cuda.current_stream()` costs several microseconds each time."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise BackendError(f"unsupported activation dtype {dtype}: float32 or bfloat16")


_device_keys: dict = {}


def device_key(device) -> str:
    """One name per CUDA device ("cuda:0"), whether it was given with or without its index."""
    key = _device_keys.get(device)
    if key is None:
        d = torch.device(device)
        if d.index is None:      # depends on the current device: not remembered
            return f"cuda:{torch.cuda.current_device()}"
        key = _device_keys[device] = f"cuda:{d.index}"
    return key


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise BackendError(f"{name} must be a CUDA tensor: there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise BackendError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() > 0 and t.stride(-1) != 1:
        raise BackendError(f"{name} must be contiguous along its last axis")


_pdl_mode = None


def set_pdl(mode: int) -> None:
    """Programmatic dependent launch: 0 off, 1 every kernel, 2 only the launches that ask for it.
    The engine switches it on for eager steps (prompts: the next kernel's CTAs start while the last
    ones of the kernel before drain, 1-3 % of a prefill) and off for steps it records as CUDA graphs
    (inside a replayed graph it measured slower); see `options.pdl_eager`."""
    global _pdl_mode
    if _pdl_mode != int(mode):
        _libmod.load().hb_set_pdl(int(mode))
        _pdl_mode = int(mode)


def set_gemm_pairs(on: bool) -> None:
    """Whether the prefill product runs as pairs of CTAs (cta_group::2) where that applies (default on)."""
    _libmod.load().hb_gemm_tcgen05_set_pairs(1 if on else 0)


def set_gemm_ksplit(on: bool) -> None:
    """Whether products of at most 128 rows cut K over a cluster of CTAs where that applies (default on)."""
    _libmod.load().hb_gemm_tcgen05_set_ksplit(1 if on else 0)


def is_available() -> bool:
    """True when a CUDA device is present (the kernels still have to build and load)."""
    return torch.cuda.is_available()


# ---------------------------------------------------------------------------------------------
def rng_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * normal(key, i): the same bits as `weights.counter_rng.normal`."""
    _check(out, None, "out")
    if not out.is_contiguous():
        raise BackendError("rng_normal: out must be contiguous")
    _run("hb_rng_normal", dtype_code(out.dtype), out.data_ptr(), out.numel(), int(key) & ((1 << 64) - 1),
         float(mean), float(std), _stream())


def fill(out: torch.Tensor, value: float) -> None:
    """Every element of a contiguous float32, bfloat16 or int32 tensor becomes `value`."""
    _check(out, None, "out")
    if not out.is_contiguous():
        raise BackendError("fill: out must be contiguous")
    code = 2 if out.dtype == torch.int32 else dtype_code(out.dtype)
    _run("hb_fill", code, out.data_ptr(), out.numel(), float(value), _stream())


_CAST_SRC = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def cast(src: torch.Tensor, dtype: torch.dtype, round_bf16: bool = False) -> torch.Tensor:
    """`src` (float32, bfloat16 or float16, contiguous, on the device) as a new tensor of `dtype`
    (float32 or bfloat16; float32 -> bfloat16 rounds to nearest even).  With `round_bf16` the
    values pass through bfloat16 whatever `dtype` is.  Returns `src` itself when nothing changes."""
    _check(src, None, "src")
    if src.dtype not in _CAST_SRC:
        raise BackendError(f"cast: cannot read {src.dtype}")
    if src.dtype == dtype and (not round_bf16 or dtype == torch.bfloat16):
        return src
    if not src.is_contiguous():
        raise BackendError("cast: src must be contiguous")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _run("hb_cast", _CAST_SRC[src.dtype], src.data_ptr(), dtype_code(dtype), out.data_ptr(), src.numel(),
         1 if round_bf16 else 0, _stream())
    return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
          pos_table: torch.Tensor | None = None, positions: torch.Tensor | None = None) -> None:
    """out[t, :] = float(table[ids[t], :]) * scale (+ float(pos_table[positions[t], :]) with a table of
    learned position vectors, in the embedding's dtype); out is the float residual stream [T, H]."""
    _check(table, None, "table"); _check(ids, torch.int32, "ids"); _check(out, torch.float32, "out")
    if pos_table is not None:
        _check(pos_table, table.dtype, "pos_table"); _check(positions, torch.int32, "positions")
        if pos_table.shape[1] != table.shape[1] or not pos_table.is_contiguous():
            raise BackendError("embed: the position table must be contiguous and as wide as the embedding")
    _run("hb_embed", dtype_code(table.dtype), table.data_ptr(), ids.data_ptr(), out.data_ptr(),
         ids.numel(), table.shape[1], table.shape[0], float(scale), _ptr(pos_table),
         _ptr(positions) if pos_table is not None else None, 0 if pos_table is None else pos_table.shape[0], _stream())


def scaled_residual_norm(y: torch.Tensor, mult: float, x: torch.Tensor, w: torch.Tensor | None = None,
                         h: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """x += mult * y (float); with w and h: h = x / sqrt(mean(x^2) + eps) * w of the updated rows, in h's dtype."""
    _check(y, torch.float32, "y"); _check(x, torch.float32, "x")
    if not x.is_contiguous() or (h is not None and not h.is_contiguous()):
        raise BackendError("scaled_residual_norm: x and h must be contiguous")
    if w is not None:
        _check(w, torch.float32, "w"); _check(h, None, "h")
    _run("hb_scaled_residual_norm", dtype_code(h.dtype) if h is not None else F32, y.data_ptr(), y.stride(0), float(mult),
         x.data_ptr(), _ptr(w), _ptr(h), x.shape[0], x.shape[1], float(eps), _stream())


def qk_prepare_cache(rows, bias, q_out, temp_coef, temp_every, tok_seq, tok_pos, seq_pages, k_cache, v_cache, num_heads,
                     num_kv_heads, head_dim, page_size, write_cache=True) -> None:
    """Float rows [q heads | k heads (| v heads)] of a projection: biases added (bias in the row's layout, or
    None), q times 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: no temperature) into
    q_out, k (and v, if a value plane is given) into the paged cache at the token's place."""
    _check(rows, torch.float32, "rows"); _check(q_out, k_cache.dtype, "q_out")
    if bias is not None:
        _check(bias, torch.float32, "bias")
    _run("hb_qk_prepare_cache", dtype_code(q_out.dtype), rows.data_ptr(), rows.stride(0), _ptr(bias), q_out.data_ptr(),
         q_out.stride(0), float(temp_coef), int(temp_every), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), k_cache.data_ptr(), _ptr(v_cache), rows.shape[0], int(num_heads), int(num_kv_heads),
         int(head_dim), int(page_size), 1 if write_cache else 0, _stream())


def to_activation(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float, contiguous) in out's dtype, rounded to nearest even: what a sublayer that reads
    the residual stream itself gets on the bfloat16 path."""
    _check(x, torch.float32, "x"); _check(out, None, "out")
    if not (x.is_contiguous() and out.is_contiguous() and x.numel() == out.numel()):
        raise BackendError("to_activation: x and out must be contiguous and of one size")
    _run("hb_cast", 0, x.data_ptr(), dtype_code(out.dtype), out.data_ptr(), x.numel(), 0, _stream())


def layernorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = (x - mean) / sqrt(var + eps) * w of row rows[r] (or r) of x; x and w float."""
    _check(x, torch.float32, "x"); _check(w, torch.float32, "w"); _check(out, None, "out")
    _run("hb_layernorm", dtype_code(out.dtype), x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(rows),
         out.shape[0], x.shape[-1], float(eps), _stream())


def layernorm_residual(y: torch.Tensor, w: torch.Tensor, scale: torch.Tensor | None, x: torch.Tensor,
                       h: torch.Tensor | None, eps: float, dtype: torch.dtype) -> None:
    """x += layernorm(y) * w * scale (scale may be None); h, if given, receives the updated x in the
    activation dtype `dtype`."""
    _check(y, torch.float32, "y"); _check(w, torch.float32, "w"); _check(x, torch.float32, "x")
    if h is not None:
        _check(h, dtype, "h")
    if not x.is_contiguous() or (h is not None and not h.is_contiguous()):
        raise BackendError("layernorm_residual: x and h must be contiguous")
    _run("hb_layernorm_residual", dtype_code(dtype), y.data_ptr(), y.stride(0), w.data_ptr(), _ptr(scale), x.data_ptr(),
         _ptr(h), x.shape[0], x.shape[1], float(eps), _stream())


def latent_kv_store(kv, norm_w, eps, freq, mscale, rank, rot, tok_seq, tok_pos, seq_pages, cache, page_size) -> None:
    """Rows [c | r] of kv (float, [T, >= rank + rot]): c normed (RMS, weight norm_w), r rotated at the
    token's position; both stored at the token's place of the one-plane paged cache."""
    _check(kv, torch.float32, "kv"); _check(norm_w, torch.float32, "norm_w"); _check(freq, torch.float32, "freq")
    _run("hb_latent_kv_store", dtype_code(cache.dtype), kv.data_ptr(), kv.stride(0), norm_w.data_ptr(), float(eps),
         freq.data_ptr(), float(mscale), int(rank), int(rot), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), cache.data_ptr(), kv.shape[0], int(page_size), _stream())


def rotate_heads(src, src_head_stride, src_offset, out, out_head_stride, out_offset, freq, mscale, tok_pos, heads, rot,
                 scale=1.0) -> None:
    """out[t, h*out_head_stride + out_offset + ..rot] = scale * rotation of src[t, h*src_head_stride + src_offset + ..rot]
    at position tok_pos[t] (pairs (i, i + rot/2), angle p * freq[i], cos and sin times mscale)."""
    _check(src, torch.float32, "src"); _check(out, torch.float32, "out"); _check(freq, torch.float32, "freq")
    _run("hb_rotate_heads", src.data_ptr(), src.stride(0), int(src_head_stride), int(src_offset), out.data_ptr(), out.stride(0),
         int(out_head_stride), int(out_offset), freq.data_ptr(), float(mscale), tok_pos.data_ptr(), src.shape[0], int(heads),
         int(rot), float(scale), _stream())


def headwise_gemm(src, src_head_stride, w, out, out_head_stride, scale=1.0, gate=None) -> None:
    """out[t, h*out_head_stride + n] = scale * sum_k src[t, h*src_head_stride + k] * w[h, n, k], times
    sigmoid(gate[t, h*N + n]) if a gate (float) is given.  src float; w [H, N, K] in the compute dtype; out
    float or the compute dtype."""
    _check(src, torch.float32, "src"); _check(w, None, "w"); _check(out, None, "out")
    if not w.is_contiguous() or w.dim() != 3:
        raise BackendError("headwise_gemm: w must be a contiguous [heads, N, K] tensor")
    if gate is not None:
        _check(gate, torch.float32, "gate")
    H, N, K = w.shape
    _run("hb_headwise_gemm", dtype_code(w.dtype), dtype_code(out.dtype), src.data_ptr(), src.stride(0), int(src_head_stride),
         w.data_ptr(), out.data_ptr(), out.stride(0), int(out_head_stride), _ptr(gate), 0 if gate is None else gate.stride(0),
         src.shape[0], H, K, N, float(scale), _stream())


def latent_attention(q, out, cache, sink, tok_seq, tok_pos, seq_pages, heads, rank, rot, page_size, window, batch=None,
                     scratch=None) -> None:
    """out[t, h, :rank] = sum_j p_j c_j over the cached rows [c_j | r_j] that the token may see, with
    scores q[t, h, :] . [c_j | r_j] (q float, already scaled) and a softmax whose denominator also holds
    exp(sink[h]) when a sink is given.  With the step's `batch` and a bfloat16 cache whose sizes the
    tensor-core kernel serves, that kernel runs; else the any-shape kernel.  A step with too few (token,
    head) rows to fill the GPU cuts every row's keys into ranges (partial results in `scratch(shape, dtype)`,
    joined by a second kernel), as many as the table of pages can hold tiles of, at most `latent_max_splits`."""
    _check(q, torch.float32, "q"); _check(out, torch.float32, "out")
    if sink is not None:
        _check(sink, torch.float32, "sink")
    if batch is not None and cache.dtype == torch.bfloat16 and options.latent_attention == "mma" \
            and _fn("hb_latent_attention_mma_ok")(int(rank), int(rot)):
        ctas = batch.n_seqs * -(-batch.max_q_len * int(heads) // 32)
        tiles = -(-min(seq_pages.shape[1] * int(page_size), int(window) + batch.max_q_len if window else 1 << 30) // 64)
        nsplit = 1
        if scratch is not None and 2 * ctas <= sm_count(out.device):
            nsplit = max(1, min(sm_count(out.device) // ctas, tiles, options.latent_max_splits))
        part = None
        if nsplit > 1:
            part = scratch((batch.n_seqs * -(-batch.max_q_len * int(heads) // 32) * nsplit * 32 * (int(rank) + 2),), torch.float32)
        _KERNELS_PER_CALL["hb_latent_attention_mma_bf16"] = 2 if nsplit > 1 else 1
        _run("hb_latent_attention_mma_bf16", q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), cache.data_ptr(),
             _ptr(sink), batch.seq_start.data_ptr(), batch.seq_pos0.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
             batch.n_seqs, batch.max_q_len, int(heads), int(rank), int(rot), int(page_size), int(window or 0), nsplit,
             _ptr(part), _stream())
        return
    _run("hb_latent_attention", dtype_code(cache.dtype), q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0),
         cache.data_ptr(), _ptr(sink), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
         q.shape[0], int(heads), int(rank), int(rot), int(page_size), int(window or 0), _stream())


def gla_decay(low, w2, bias, tau, out) -> None:
    """out[t, c] = sigmoid(z)^(1/tau) with z = bias[c] + low[t, :] . w2[c, :]; low and out float."""
    _check(low, torch.float32, "low"); _check(w2, None, "w2"); _check(out, torch.float32, "out")
    _run("hb_gla_decay", dtype_code(w2.dtype), low.data_ptr(), low.stride(0), w2.data_ptr(), _ptr(bias), 1.0 / float(tau),
         out.data_ptr(), low.shape[0], w2.shape[0], w2.shape[1], _stream())


def gla_scan(proj, q_off, k_off, v_off, decay, state, seq_slot, seq_start, out, n_seqs, heads, dk, dv, qscale) -> None:
    """The recurrence S = diag(a) S + k v^T, o = S^T (q * qscale) over every sequence's tokens of the step, in
    order, from and into state[slot] ([slots, heads, dk, dv] float).  q, k, v are column ranges of proj."""
    _check(proj, torch.float32, "proj"); _check(decay, torch.float32, "decay"); _check(state, torch.float32, "state")
    _check(out, torch.float32, "out")
    if not (state.is_contiguous() and decay.is_contiguous()):
        raise BackendError("gla_scan: state and decay must be contiguous")
    _run("hb_gla_scan", proj.data_ptr(), proj.stride(0), int(q_off), int(k_off), int(v_off), decay.data_ptr(), state.data_ptr(),
         seq_slot.data_ptr(), seq_start.data_ptr(), out.data_ptr(), out.stride(0), int(n_seqs), int(heads), int(dk), int(dv),
         float(qscale), _stream())


def gla_output(o, w, eps, gate, out, heads, dv) -> None:
    """out[t, h, :] = rmsnorm(o[t, h, :]) * w * silu(gate[t, h, :]); o and gate float, out in the activation dtype."""
    _check(o, torch.float32, "o"); _check(w, torch.float32, "w"); _check(gate, torch.float32, "gate"); _check(out, None, "out")
    _run("hb_gla_output", dtype_code(out.dtype), o.data_ptr(), o.stride(0), w.data_ptr(), float(eps), gate.data_ptr(),
         gate.stride(0), out.data_ptr(), out.stride(0), o.shape[0], int(heads), int(dv), _stream())


def group_rmsnorm(x, w, out, eps, groups=1, rows=None) -> None:
    """out[r] = row rows[r] (or r) of x, cut into `groups` equal consecutive parts, each divided by its own
    sqrt(mean(part^2) + eps), the whole times w; x and w float, out in its own dtype."""
    _check(x, torch.float32, "x"); _check(w, torch.float32, "w"); _check(out, None, "out")
    if not (x.is_contiguous() and out.is_contiguous()):
        raise BackendError("group_rmsnorm: x and out must be contiguous")
    _run("hb_group_rmsnorm", dtype_code(out.dtype), x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(rows), out.shape[0],
         x.shape[-1], int(groups), float(eps), _stream())


def group_rmsnorm_residual(y, w, x, h, eps, groups, dtype, bias=None, second=None) -> None:
    """x += GN(y + bias) * w with GN the RMS norm in `groups` parts (bias [D] float or None); h, if given,
    receives the updated x in the activation dtype `dtype`.  With `second` = (z, a, b) the normed vector is
    a * y + b * z + bias (z float, of y's shape)."""
    _check(y, torch.float32, "y"); _check(w, torch.float32, "w"); _check(x, torch.float32, "x")
    if h is not None:
        _check(h, dtype, "h")
    if bias is not None:
        _check(bias, torch.float32, "bias")
    if not x.is_contiguous() or (h is not None and not h.is_contiguous()):
        raise BackendError("group_rmsnorm_residual: x and h must be contiguous")
    z, a, b = second if second is not None else (None, 1.0, 0.0)
    if z is not None:
        _check(z, torch.float32, "z")
        if z.shape != y.shape:
            raise BackendError("group_rmsnorm_residual: the second array must have the first one's shape")
    _run("hb_group_rmsnorm_residual", dtype_code(dtype), y.data_ptr(), y.stride(0), _ptr(z), z.stride(0) if z is not None else 0,
         float(a), float(b), _ptr(bias), w.data_ptr(), x.data_ptr(), _ptr(h), x.shape[0], x.shape[1], int(groups), float(eps),
         _stream())


def axpby(y, a, z, b) -> None:
    """y = a * y + b * z, float arrays of one shape (rows may be strided)."""
    _check(y, torch.float32, "y"); _check(z, torch.float32, "z")
    if y.shape != z.shape:
        raise BackendError("axpby: y and z must have one shape")
    _run("hb_axpby", y.data_ptr(), y.stride(0), float(a), z.data_ptr(), z.stride(0), float(b), y.shape[0], y.shape[1], _stream())


def add_row_bias(y, bias) -> None:
    """y[r, :] += bias for every row (float)."""
    _check(y, torch.float32, "y"); _check(bias, torch.float32, "bias")
    if bias.numel() != y.shape[1]:
        raise BackendError("add_row_bias: the bias must have one number per column")
    _run("hb_axpby", y.data_ptr(), y.stride(0), 1.0, bias.data_ptr(), 0, 1.0, y.shape[0], y.shape[1], _stream())


def bias_glu(gu, bias, out, interleave, act) -> None:
    """out = act(gate + b) * (up + b) from float sums gu [T, 2 inter] (bias in gu's column layout, or None)."""
    _check(gu, torch.float32, "gu"); _check(out, None, "out")
    if bias is not None:
        _check(bias, torch.float32, "bias")
    _run("hb_bias_glu", dtype_code(out.dtype), gu.data_ptr(), gu.stride(0), _ptr(bias), out.data_ptr(), out.stride(0),
         gu.shape[0], out.shape[1], int(interleave), int(act), _stream())


def tanh_cap(x, cap) -> None:
    """x <- cap * tanh(x / cap), float, in place."""
    _check(x, torch.float32, "x")
    _run("hb_tanh_cap", x.data_ptr(), x.stride(0), float(cap), x.shape[0], x.shape[1], _stream())


def short_conv(inp, w, state, batch, out, add_input=False, silu=False) -> None:
    """A causal convolution over time per channel: out_t = (in_t +) sum_j w[:, j] in_{t - taps + 1 + j} (then silu);
    inp float [T, C] (rows may be strided), w float [C, taps], state float [slots, taps - 1, C] (the sequence's
    last inputs: read for a step's first tokens, then replaced by the step's last inputs), out [T, C] in its dtype."""
    _check(inp, torch.float32, "inp"); _check(w, torch.float32, "w"); _check(out, None, "out")
    taps = w.shape[1]
    if state is not None:
        _check(state, torch.float32, "state")
        if not state.is_contiguous() or tuple(state.shape[1:]) != (taps - 1, inp.shape[1]):
            raise BackendError(f"short_conv: state of shape {tuple(state.shape)} does not hold {taps - 1} inputs of {inp.shape[1]} channels")
    if not w.is_contiguous():
        raise BackendError("short_conv: w must be contiguous")
    _run("hb_short_conv", dtype_code(out.dtype), inp.data_ptr(), inp.stride(0), w.data_ptr(), _ptr(state),
         batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(), batch.seq_pos0.data_ptr(), out.data_ptr(), out.stride(0),
         batch.n_seqs, batch.max_q_len, inp.shape[1], taps, 1 if add_input else 0, 1 if silu else 0, _stream())


def pair_embed(table, pair_table, batch, last_id, out, buckets, mul_prev, mul_cur, scale=1.0) -> None:
    """out[t] = table[id_t] * scale + pair_table[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets] (row `buckets`
    for a sequence's first token); the id before a step's first token is last_id[slot] (int32 [slots, 1]), where
    the step then leaves its own last id."""
    _check(table, None, "table"); _check(pair_table, table.dtype, "pair_table"); _check(out, torch.float32, "out")
    _check(last_id, torch.int32, "last_id")
    if pair_table.shape != (buckets + 1, table.shape[1]) or not pair_table.is_contiguous():
        raise BackendError(f"pair_embed: the pair table must be [{buckets + 1}, {table.shape[1]}] and contiguous")
    _run("hb_pair_embed", dtype_code(table.dtype), table.data_ptr(), pair_table.data_ptr(), batch.token_ids.data_ptr(),
         batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(),
         last_id.data_ptr(), out.data_ptr(), batch.n_tokens, table.shape[1], table.shape[0], int(buckets), int(mul_prev),
         int(mul_cur), float(scale), _stream())


def silu_columns(x, col0, cols) -> None:
    """x[:, col0:col0 + cols] <- silu of it, float, in place."""
    _check(x, torch.float32, "x")
    _run("hb_silu_columns", x.data_ptr(), x.stride(0), int(col0), int(cols), x.shape[0], _stream())


def delta_prepare(qk, q_off, k_off, qk_heads, dk, qscale, ab, b_off, a_off, a_log, dt_bias, gates, heads) -> None:
    """In place on float rows qk: every q and k head (column ranges from q_off, k_off) becomes x / sqrt(sum x^2 + 1e-6),
    q also times qscale.  gates [T, 2 heads] float: g = exp(-exp(a_log) softplus(ab[:, a_off + h] + dt_bias)), then
    beta = sigmoid(ab[:, b_off + h])."""
    for t, n in ((qk, "qk"), (ab, "ab"), (a_log, "a_log"), (dt_bias, "dt_bias"), (gates, "gates")):
        _check(t, torch.float32, n)
    if not gates.is_contiguous():
        raise BackendError("delta_prepare: gates must be contiguous")
    _run("hb_delta_prepare", qk.data_ptr(), qk.stride(0), int(q_off), int(k_off), int(qk_heads), int(dk), float(qscale),
         ab.data_ptr(), ab.stride(0), int(b_off), int(a_off), a_log.data_ptr(), dt_bias.data_ptr(), gates.data_ptr(),
         int(heads), qk.shape[0], _stream())


def linear_scan(q, k, v, state, batch, out, heads, qk_heads, dk, dv, gates=None, decay=None) -> None:
    """The recurrence of a matrix state per head over every sequence's tokens of the step, in order, from and into
    state[slot] ([slots, heads, dk, dv] float).  With `gates` ([T, 2 heads]: g, beta) the gated delta rule
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; with `decay` ([heads]) S <- d S + k v^T.  o = S^T q.
    q, k [T, qk_heads dk], v and out [T, heads dv]: float column ranges of rows."""
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (state, "state"), (out, "out")):
        _check(t, torch.float32, n)
    if not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dk, dv):
        raise BackendError(f"linear_scan: state of shape {tuple(state.shape)} is not [slots, {heads}, {dk}, {dv}]")
    if (gates is None) == (decay is None):
        raise BackendError("linear_scan: give the delta rule's gates or the constant decays")
    _run("hb_linear_scan", 1 if gates is not None else 0, q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
         v.stride(0), _ptr(gates), _ptr(decay), state.data_ptr(), batch.seq_slot.data_ptr(), batch.seq_start.data_ptr(),
         out.data_ptr(), out.stride(0), batch.n_seqs, batch.max_q_len, int(heads), int(qk_heads), int(dk), int(dv), _stream())


def gated_rmsnorm(o, w, eps, gate, out, units, n, sigmoid_gate=False) -> None:
    """out[t, u, :] = o[t, u, :] / sqrt(mean(o[t, u, :]^2) + eps) * w * act(gate[t, u, :]) for `units` runs of n columns;
    w [n] is shared by the units (units == 1: one norm over the whole row), or w [units * n] has a part for each.
    act: silu, or the sigmoid."""
    _check(o, torch.float32, "o"); _check(w, torch.float32, "w"); _check(gate, torch.float32, "gate"); _check(out, None, "out")
    if w.numel() not in (n, units * n):
        raise BackendError(f"gated_rmsnorm: the weight has {w.numel()} numbers, a unit {n}, all units {units * n}")
    _run("hb_gated_rmsnorm", dtype_code(out.dtype), o.data_ptr(), o.stride(0), w.data_ptr(), float(eps), gate.data_ptr(),
         gate.stride(0), out.data_ptr(), out.stride(0), o.shape[0], int(units), int(n), 1 if sigmoid_gate else 0,
         int(n) if (units > 1 and w.numel() == units * n) else 0, _stream())


def qkv_rotary_cache(rows, wq, wk, eps, fqk, rot, halves, fv, batch, seq_pages, q_out, k_cache, v_cache, num_heads,
                     num_kv_heads, dk, dv, hd, page_size, write_cache=True) -> None:
    """Float rows [q: heads x dk | k: kv heads x dk | v: kv heads x dv]: q and k normed over the whole projection
    (weights wq, wk; None: no norm), pair m of their first `rot` channels turned by p * fqk[m], pair m of all value
    channels by p * fv[m] (fv None: values as they are); q into q_out (heads of hd channels), k and v into the paged
    cache (heads of hd channels, zeros beyond dk and dv)."""
    _check(rows, torch.float32, "rows"); _check(q_out, k_cache.dtype, "q_out")
    for t, n in ((wq, "wq"), (wk, "wk"), (fqk, "fqk"), (fv, "fv")):
        if t is not None:
            _check(t, torch.float32, n)
    _run("hb_qkv_rotary_cache", dtype_code(q_out.dtype), rows.data_ptr(), rows.stride(0), _ptr(wq), _ptr(wk), float(eps),
         1 if wq is not None else 0, _ptr(fqk), int(rot), 1 if halves else 0, _ptr(fv), batch.tok_seq.data_ptr(),
         batch.tok_pos.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0), q_out.data_ptr(), q_out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), rows.shape[0], int(num_heads), int(num_kv_heads), int(dk), int(dv), int(hd),
         int(page_size), 1 if write_cache else 0, _stream())


def rotate_heads_back(att, hd, fv, halves, tok_pos, out, num_heads, dv) -> None:
    """out[t, h, :dv] = the first dv channels of head h of att (heads of hd channels), pair m turned by -p * fv[m]
    (fv None: copied)."""
    _check(att, out.dtype, "att")
    _run("hb_rotate_heads_back", dtype_code(out.dtype), att.data_ptr(), att.stride(0), int(hd), _ptr(fv), 1 if halves else 0,
         tok_pos.data_ptr(), out.data_ptr(), out.stride(0), att.shape[0], int(num_heads), int(dv), _stream())


def head_gate(att, hd, gate, out, num_heads, dv) -> None:
    """out[t, h, :dv] = the first dv channels of head h of att (heads of hd channels) times sigmoid(gate[t, h]);
    gate float [T, num_heads] (rows may be strided), or None: the channels as they are."""
    _check(att, out.dtype, "att")
    if gate is not None:
        _check(gate, torch.float32, "gate")
    _run("hb_head_gate", dtype_code(out.dtype), att.data_ptr(), att.stride(0), int(hd), _ptr(gate), gate.stride(0) if gate is not None else 0,
         out.data_ptr(), out.stride(0), att.shape[0], int(num_heads), int(dv), _stream())


def general_delta_prepare(rows, r_off, k_off, a_off, low_off, w2, w0, a0, decay_c, unit_eps, prep, heads, dk) -> None:
    """From float rows of a projection (column ranges r, k, a of heads * dk numbers from their offsets, the decay's
    inner row of w2.shape[1] numbers from low_off): prep [T, heads, 5, dk] float = r, k, w, u, a * u with
    u = k / sqrt(sum k^2 + unit_eps) per head, w = exp(-decay_c * sigmoid(w2 tanh(low) + w0)), a = sigmoid(a + a0)."""
    _check(rows, torch.float32, "rows"); _check(w2, None, "w2"); _check(w0, torch.float32, "w0"); _check(a0, torch.float32, "a0")
    _check(prep, torch.float32, "prep")
    if not (w2.is_contiguous() and prep.is_contiguous()) or tuple(w2.shape[:1]) != (heads * dk,):
        raise BackendError("general_delta_prepare: w2 must be [heads * dk, rank] and contiguous, prep contiguous")
    _run("hb_general_delta_prepare", dtype_code(w2.dtype), rows.data_ptr(), rows.stride(0), int(r_off), int(k_off), int(a_off),
         int(low_off), w2.data_ptr(), w0.data_ptr(), a0.data_ptr(), float(decay_c), float(unit_eps), prep.data_ptr(),
         rows.shape[0], int(heads), int(dk), w2.shape[1], _stream())


def general_delta_scan(prep, v, state, batch, out, heads, dk, dv) -> None:
    """The generalised delta rule over every sequence's tokens of the step, in order, from and into state[slot]
    ([slots, heads, dk, dv] float): S <- diag(w) S - (a u) (u^T S) + k v^T (both terms read the old S); o = S^T r.
    prep [T, heads, 5, dk] as `general_delta_prepare` leaves it; v and out [T, heads dv] float column ranges of rows."""
    for t, n in ((prep, "prep"), (v, "v"), (state, "state"), (out, "out")):
        _check(t, torch.float32, n)
    if not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dk, dv):
        raise BackendError(f"general_delta_scan: state of shape {tuple(state.shape)} is not [slots, {heads}, {dk}, {dv}]")
    _run("hb_general_delta_scan", prep.data_ptr(), v.data_ptr(), v.stride(0), state.data_ptr(), batch.seq_slot.data_ptr(),
         batch.seq_start.data_ptr(), out.data_ptr(), out.stride(0), batch.n_seqs, int(heads), int(dk), int(dv), _stream())


def gated_norm_residual(y, w, eps, x, dtype, gate=None, gate_bias=None, next_norm=None, h=None) -> None:
    """x += v / sqrt(mean(v^2) + eps) * w with v = y * sigmoid(gate + gate_bias) (gate None: v = y); all float.
    h, if given, receives in the activation dtype `dtype` the updated x, or with next_norm = (w2, eps2) its RMS norm
    x / sqrt(mean(x^2) + eps2) * w2."""
    _check(y, torch.float32, "y"); _check(w, torch.float32, "w"); _check(x, torch.float32, "x")
    if gate is not None:
        _check(gate, torch.float32, "gate")
    if gate_bias is not None:
        _check(gate_bias, torch.float32, "gate_bias")
    if h is not None:
        _check(h, dtype, "h")
    if not x.is_contiguous() or (h is not None and not h.is_contiguous()):
        raise BackendError("gated_norm_residual: x and h must be contiguous")
    w2, eps2 = next_norm if next_norm is not None else (None, 0.0)
    _run("hb_gated_norm_residual", dtype_code(dtype), y.data_ptr(), y.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0,
         _ptr(gate_bias), w.data_ptr(), float(eps), x.data_ptr(), _ptr(w2), float(eps2), _ptr(h), x.shape[0], x.shape[1], _stream())


def token_gate(s, table, col0, ids, out) -> None:
    """out[t, j] = gelu_tanh(s[t, j]) * table[ids[t], col0 + j]; s float [T, m], table in out's dtype."""
    _check(s, torch.float32, "s"); _check(table, out.dtype, "table"); _check(ids, torch.int32, "ids")
    _run("hb_token_gate", dtype_code(out.dtype), s.data_ptr(), s.stride(0), table.data_ptr(), table.stride(0), int(col0),
         ids.data_ptr(), out.data_ptr(), out.stride(0), s.shape[0], s.shape[1], table.shape[0], _stream())


def moe_route(h, w_router, ids, weights, top, renorm=False, score=0, groups=1, keep=1, group_top=2, weight_scale=1.0) -> None:
    """ids[t, :top], weights[t, :top]: the `top` largest scores of w_router h[t] (ties to the lower index);
    score 0: softmax over all experts, 1: sigmoid.  With groups > 1 the experts form that many equal groups of
    neighbours, a group's score is the sum of its `group_top` largest scores, and only the experts of the
    `keep` best groups can be chosen.  The weights are the chosen scores (divided by their sum with `renorm`)
    times `weight_scale`."""
    _check(h, None, "h"); _check(w_router, h.dtype, "w_router"); _check(ids, torch.int32, "ids"); _check(weights, torch.float32, "weights")
    _run("hb_moe_route", dtype_code(h.dtype), h.data_ptr(), h.stride(0), w_router.data_ptr(), ids.data_ptr(), weights.data_ptr(),
         h.shape[0], h.shape[1], w_router.shape[0], int(top), 1 if renorm else 0, int(score), int(groups), int(keep),
         int(group_top), float(weight_scale), _stream())


MOE_GROUPED_MIN_TOKENS = 32


MOE_TC_MIN_PAIRS = 512
GATED_HALVES, GATED_GROUPS_OF_8 = 1, 2     # layouts of a gated expert's first matrix (see `moe_experts`)


def moe_grouped_ok(h, up, gated=0) -> bool:
    """Whether a step's routed feed-forward goes through the grouped tensor-core product: bfloat16, enough
    tokens that an expert's matrices are worth reading once per tile of pairs, widths in 16-byte pieces."""
    E, F, D = up.shape
    if gated:
        F //= 2
    return (options.moe_grouped and h.dtype == torch.bfloat16 and MOE_GROUPED_MIN_TOKENS <= h.shape[0] <= 65535
            and D % 8 == 0 and F % 8 == 0 and h.stride(0) % 8 == 0 and E <= 1024 and h.data_ptr() % 16 == 0
            and gated in (0, GATED_GROUPS_OF_8))


def moe_tc_ok(h, up, top, gated, act) -> bool:
    """Whether the grouped products run on tcgen05: what `moe_grouped_ok` asks, gated experts with silu or the clamped
    activation (the product's fused epilogue), and enough (token, expert) pairs that tiles of 128 rows per expert fill."""
    return (options.moe_tc and moe_grouped_ok(h, up, gated) and gated == GATED_GROUPS_OF_8 and act in (ACT_SILU, ACT_SWISH_CLAMP)
            and h.shape[0] * int(top) >= MOE_TC_MIN_PAIRS)


def moe_experts_tc(h, up, down, ids, weights, y, accumulate, scratch, act_limit=0.0) -> None:
    """moe_experts for long prompts, gated experts with silu (or, with act_limit > 0, the clamped activation): the pairs
    sorted by expert into runs padded to tiles of 128 rows, both products on tcgen05 (the first with the gated
    activation in its epilogue)."""
    _check(h, torch.bfloat16, "h"); _check(up, torch.bfloat16, "up"); _check(down, torch.bfloat16, "down"); _check(y, torch.float32, "y")
    T, top = ids.shape
    E, F2, D = up.shape
    F = F2 // 2
    rows = int(_fn("hb_moe_experts_tc_rows")(T, E, top))
    if rows <= 0:
        raise BackendError("moe_experts_tc: too many (token, expert) pairs")
    ints = scratch((T * top + rows // 128 + 1,), torch.int32)
    srt = scratch((rows, D), torch.bfloat16)
    mid = scratch((rows, F), torch.bfloat16)
    part = scratch((rows, D), torch.float32)
    _tcgen05_workspace(y.device)
    _run("hb_moe_experts_tc_bf16", h.data_ptr(), h.stride(0), up.data_ptr(), down.data_ptr(), ids.data_ptr(), weights.data_ptr(),
         ints.data_ptr(), srt.data_ptr(), mid.data_ptr(), part.data_ptr(), y.data_ptr(), y.stride(0), T, D, E, F, top,
         float(act_limit), 1 if accumulate else 0, _error_flag(y.device).data_ptr(), _stream())


def moe_experts_grouped(h, up, down, ids, weights, y, act, accumulate, scratch, gated=0, act_limit=0.0) -> None:
    """moe_experts for many tokens: pairs grouped by expert on the device, tiles of 64 pairs on the tensor cores."""
    _check(h, torch.bfloat16, "h"); _check(up, torch.bfloat16, "up"); _check(down, torch.bfloat16, "down"); _check(y, torch.float32, "y")
    T, top = ids.shape
    E, F, D = up.shape
    if gated:
        F //= 2
    ints = scratch((2 * (E + 1) + T * top,), torch.int32)
    mid = scratch((T * top, F), torch.bfloat16)
    part = scratch((T * top, D), torch.float32)
    _run("hb_moe_experts_grouped_bf16", h.data_ptr(), h.stride(0), up.data_ptr(), down.data_ptr(), ids.data_ptr(), weights.data_ptr(),
         ints.data_ptr(), mid.data_ptr(), part.data_ptr(), y.data_ptr(), y.stride(0), T, D, E, F, top, int(act),
         int(gated), float(act_limit), 1 if accumulate else 0, _stream())


def moe_experts(h, up, down, ids, weights, mid, y, act, accumulate=False, gated=0, act_limit=0.0) -> None:
    """y[t] (+)= sum_r weights[t, r] * down[e] act(up[e] h[t]), e = ids[t, r]; up [E, F, D], down [E, D, F] in
    h's dtype; mid [T * top, F] scratch in h's dtype; y float.  gated: up is [E, 2F, D] and an expert is
    down[e] (act(gate h) * (up h)), with the gate and up rows in turn in groups of 8 (GATED_GROUPS_OF_8) or all
    gate rows before all up rows (GATED_HALVES).  act ACT_SWISH_CLAMP (gated experts only) takes `act_limit`."""
    _check(h, None, "h"); _check(up, h.dtype, "up"); _check(down, h.dtype, "down"); _check(mid, h.dtype, "mid"); _check(y, torch.float32, "y")
    if not (up.is_contiguous() and down.is_contiguous() and mid.is_contiguous()):
        raise BackendError("moe_experts: up, down and mid must be contiguous")
    _run("hb_moe_experts", dtype_code(h.dtype), h.data_ptr(), h.stride(0), up.data_ptr(), down.data_ptr(), ids.data_ptr(),
         weights.data_ptr(), mid.data_ptr(), y.data_ptr(), y.stride(0), h.shape[0], h.shape[1], down.shape[2], ids.shape[1],
         int(act), int(gated), float(act_limit), 1 if accumulate else 0, _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * w; x and w float, out in the activation dtype."""
    _check(x, torch.float32, "x"); _check(w, torch.float32, "w"); _check(out, None, "out")
    n = out.shape[0]
    _run("hb_rmsnorm", dtype_code(out.dtype), x.data_ptr(), w.data_ptr(), out.data_ptr(), _ptr(rows),
         n, x.shape[-1], float(eps), _stream())


def swiglu(gu: torch.Tensor, out: torch.Tensor, interleave: int, act: int = ACT_SILU) -> None:
    """out[t, i] = act(gate) * up from gu [T, 2I] (see the kernel for the column layout); act: ACT_*."""
    _check(gu, None, "gu"); _check(out, gu.dtype, "out")
    _run("hb_swiglu", dtype_code(gu.dtype), gu.data_ptr(), gu.stride(0), out.data_ptr(), out.stride(0),
         gu.shape[0], out.shape[1], int(interleave), int(act), _stream())


def add_residual(residual: torch.Tensor, y: torch.Tensor) -> None:
    """residual += y (float sum)."""
    _check(residual, torch.float32, "residual"); _check(y, None, "y")
    _run("hb_add_residual", dtype_code(y.dtype), residual.data_ptr(), y.data_ptr(), y.stride(0),
         y.shape[0], y.shape[1], _stream())


def qk_norm_rope_cache(qkv, q_weight, k_weight, eps, cos, sin, rotary_dim, tok_seq, tok_pos, seq_pages,
                       k_cache, v_cache, num_heads, num_kv_heads, head_dim, page_size, write_cache=True) -> None:
    """Head norm + rotation of q (in place) and k (into the cache), v copied into the cache."""
    _check(qkv, None, "qkv")
    _run("hb_qk_norm_rope_cache", dtype_code(qkv.dtype), qkv.data_ptr(), qkv.stride(0), _ptr(q_weight),
         _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), int(rotary_dim),
         0 if cos is None else cos.shape[0], tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), qkv.shape[0], num_heads,
         num_kv_heads, head_dim, page_size, 1 if write_cache else 0, _stream())


def gemm_simt(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T on the CUDA cores, any sizes."""
    _check(a, None, "a"); _check(w, a.dtype, "w"); _check(c, None, "c")
    _run("hb_gemm_simt", dtype_code(a.dtype), a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0),
         c.data_ptr(), c.stride(0), a.shape[0], w.shape[0], a.shape[1], epilogue, _stream())


def attention_simt(q, ldq, out, k_cache, v_cache, tok_seq, tok_pos, seq_pages, num_heads, num_kv_heads,
                   head_dim, page_size, scale, window, softcap=None, sink=None, gate_bias=None, out_gate=None) -> None:
    """Any shape, both precisions.  softcap c: score <- c * tanh(score / c); sink [num_heads] float: exp(sink)
    joins each head's softmax denominator.  v_cache may be k_cache (values that are the keys).  gate_bias
    [num_heads] float: no softmax, a visible key weighs sigmoid(score + gate_bias[head]) as it is.  out_gate
    [tokens, num_heads] float (rows may be strided): a head's result is multiplied by sigmoid(out_gate[token, head])."""
    if sink is not None:
        _check(sink, torch.float32, "sink")
    if gate_bias is not None:
        _check(gate_bias, torch.float32, "gate_bias")
    og, ldg = _out_gate(out_gate, out.shape[0], num_heads)
    _run("hb_attention_simt", dtype_code(out.dtype), q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(),
         seq_pages.stride(0), out.shape[0], num_heads, num_kv_heads, head_dim, page_size, float(scale),
         int(window or 0), float(softcap or 0.0), _ptr(sink), _ptr(gate_bias), og, ldg, _stream())


def _out_gate(out_gate, rows, num_heads):
    """(pointer, row stride) of a gate per token and head, float [rows, num_heads]; (None, 0) without one."""
    if out_gate is None:
        return None, 0
    _check(out_gate, torch.float32, "out_gate")
    if tuple(out_gate.shape) != (rows, num_heads):
        raise BackendError(f"attention: the gate per token and head must be [{rows}, {num_heads}], got {tuple(out_gate.shape)}")
    return out_gate.data_ptr(), out_gate.stride(0)


_argmax_scratch: dict = {}
ARGMAX_SCRATCH_ROWS = 4096


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of row r."""
    _check(logits, torch.float32, "logits"); _check(out, torch.int32, "out")
    key = device_key(logits.device)
    if key not in _argmax_scratch:
        _argmax_scratch[key] = torch.empty(2 * 64 * ARGMAX_SCRATCH_ROWS, dtype=torch.int32, device=logits.device)
    sc = _argmax_scratch[key]
    _run("hb_argmax", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(),
         sc.data_ptr(), sc.numel(), _stream())


_sample_flags: dict = {}


def sample(logits, temperature, top_k, top_p, uniforms, out) -> None:
    """One token per row under temperature / top-k / top-p with the row's uniform.  A small top_k
    against a large vocabulary takes a kernel that reads the row twice and works on a list of
    candidates in shared memory; rows it cannot hold fall to the general kernel in the same call."""
    _check(logits, torch.float32, "logits"); _check(uniforms, torch.float32, "uniforms"); _check(out, torch.int32, "out")
    key = device_key(logits.device)
    if key not in _sample_flags or _sample_flags[key].numel() < logits.shape[0]:
        _sample_flags[key] = torch.zeros(max(1024, logits.shape[0]), dtype=torch.int32, device=logits.device)
    _run("hb_sample", logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], float(temperature),
         int(top_k), float(top_p), uniforms.data_ptr(), out.data_ptr(), _sample_flags[key].data_ptr(), _stream())


def gemm_skinny(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T for at most 64 rows of a (bfloat16), streaming w once; EPI_SWIGLU: w holds
    gate/up rows in groups of 8 and c is [M, N/2]."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    _run("hb_gemm_skinny_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, _stream())


SHARED_NORM_MAX_ROWS = 16


class PendingNorm:
    """An RMSNorm that the product before it has begun and the product after it will finish.

    `xw` [T, D] is x * w in bfloat16; `sumsq` [parts, stride] holds partial sums of x^2 per row, so
    that y = xw / sqrt(sum(sumsq[:, row]) / D + eps).  A product kernel that takes it multiplies its
    results by that row factor; `finish_norm` makes the plain y for anyone else."""

    __slots__ = ("xw", "sumsq", "parts", "eps")

    def __init__(self, xw, sumsq, parts, eps):
        self.xw, self.sumsq, self.parts, self.eps = xw, sumsq, parts, eps

    stride = property(lambda self: self.sumsq.stride(0))

    shape = property(lambda self: self.xw.shape)
    dtype = property(lambda self: self.xw.dtype)


def shared_norm_ok(n_rows: int, dtype, dim: int) -> bool:
    """Whether products of `n_rows` activation rows can carry a norm over `dim` between them: the
    mma.sync kernel can for at most 16 rows, the tensor-memory kernel for any number; between 17
    and 64 rows a product that goes through another kernel leaves the norm to a kernel of its own."""
    return options.shared_norm and dtype == torch.bfloat16 and dim % 8 == 0


def finish_norm(p: PendingNorm, out: torch.Tensor) -> None:
    _check(out, torch.bfloat16, "out")
    _run("hb_finish_norm", p.xw.data_ptr(), p.xw.stride(0), p.sumsq.data_ptr(), p.parts, p.stride, float(p.eps),
         out.data_ptr(), out.stride(0), p.xw.shape[0], p.xw.shape[1], _stream())


def gemm_skinny_norm(a, w, c, epilogue=EPI_STORE, next_norm=None, scratch=None):
    """gemm_skinny with a norm shared on either side (at most 16 rows).  `a` may be a PendingNorm.
    next_norm = (weight [N] float, eps) with EPI_RESIDUAL: returns the PendingNorm of the updated c,
    its buffers taken from `scratch(shape, dtype)`."""
    pend = a if isinstance(a, PendingNorm) else None
    x = pend.xw if pend is not None else a
    _check(x, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    M, N, K = x.shape[0], w.shape[0], x.shape[1]
    out = None
    if next_norm is not None:
        nw, eps = next_norm
        _check(nw, torch.float32, "next norm weight")
        if epilogue != EPI_RESIDUAL or nw.numel() != N:
            raise BackendError("gemm_skinny_norm: the next norm needs the residual epilogue and a weight per output column")
        parts = int(_fn("hb_gemm_skinny_norm_parts")(M, N))
        out = PendingNorm(scratch((M, N), torch.bfloat16), scratch((parts, 16), torch.float32), parts, eps)
    _run("hb_gemm_skinny_norm_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         M, N, K, epilogue,
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         float(pend.eps) if pend is not None else 0.0,
         nw.data_ptr() if out is not None else None,
         out.xw.data_ptr() if out is not None else None, out.xw.stride(0) if out is not None else 0,
         out.sumsq.data_ptr() if out is not None else None, _stream())
    return out


_error_flags: dict = {}


def _error_flag(device) -> torch.Tensor:
    """One int per device that kernels with bounded waits set when a wait runs out."""
    key = device_key(device)
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_kernel_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check (reads one int per device,
    which waits for the device)."""
    for key, flag in _error_flags.items():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            # a kernel that gave up may have left arrival counters mid-count: start them afresh
            for table in (_decode_counters, _work_counters):
                if key in table:
                    table[key].zero_()
            if _tcgen05_ws.get(key) is not None:
                _tcgen05_ws[key][1].zero_()
            if key in _stream_bufs:
                _stream_bufs[key][1].zero_()
            raise BackendError(f"a kernel on {key} gave up waiting on a barrier (code {code}); its output is not valid")


_tcgen05_ws: dict = {}


def _tcgen05_workspace(device) -> None:
    """Once per device: hand the prefill product the workspace in which CTAs that share an output
    tile leave their pieces (about 39 MB on 148 SMs)."""
    key = device_key(device)
    if key in _tcgen05_ws:
        return
    if not options.prefill_split_tiles:
        _tcgen05_ws[key] = None
        return
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    lib = _libmod.load()
    lib.hb_gemm_tcgen05_workspace_floats.restype = ctypes.c_longlong
    lib.hb_gemm_tcgen05_workspace_floats.argtypes = [c_int]
    n = int(lib.hb_gemm_tcgen05_workspace_floats(sms))
    floats = torch.empty(n, dtype=torch.float32, device=device)
    counters = torch.zeros(sms, dtype=torch.int32, device=device)
    lib.hb_gemm_tcgen05_set_workspace.argtypes = [c_void_p, c_void_p, c_int]
    lib.hb_gemm_tcgen05_set_workspace.restype = c_int
    lib.hb_gemm_tcgen05_set_workspace(floats.data_ptr(), counters.data_ptr(), sms)
    _tcgen05_ws[key] = (floats, counters)


def gemm_tcgen05(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T on tcgen05 tensor cores with TMA-fed tiles (bfloat16, K a multiple of 8)."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    _tcgen05_workspace(c.device)
    _run("hb_gemm_tcgen05_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, _error_flag(a.device).data_ptr(), _stream())


_stream_bufs: dict = {}
STREAM_COUNTERS = 8192


def gemm_tcgen05_norm(a, w, c, epilogue=EPI_STORE, next_norm=None, scratch=None):
    """gemm_tcgen05 with a norm shared on either side (see gemm_skinny_norm): `a` may be a
    PendingNorm; next_norm = (weight, eps) with EPI_RESIDUAL returns the PendingNorm of the updated c."""
    pend = a if isinstance(a, PendingNorm) else None
    x = pend.xw if pend is not None else a
    _check(x, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    M, N, K = x.shape[0], w.shape[0], x.shape[1]
    out, nw = None, None
    if next_norm is not None:
        nw, eps = next_norm
        _check(nw, torch.float32, "next norm weight")
        if epilogue != EPI_RESIDUAL or nw.numel() != N:
            raise BackendError("gemm_tcgen05_norm: the next norm needs the residual epilogue and a weight per output column")
        parts = int(_fn("hb_gemm_tcgen05_norm_parts")(M, N))
        out = PendingNorm(scratch((M, N), torch.bfloat16), scratch((parts, (M + 3) // 4 * 4), torch.float32), parts, eps)
    _tcgen05_workspace(c.device)
    _run("hb_gemm_tcgen05_norm_bf16", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         M, N, K, epilogue,
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         pend.stride if pend is not None else 0, float(pend.eps) if pend is not None else 0.0,
         nw.data_ptr() if out is not None else None, out.xw.data_ptr() if out is not None else None,
         out.xw.stride(0) if out is not None else 0, out.sumsq.data_ptr() if out is not None else None,
         out.stride if out is not None else 0, _error_flag(c.device).data_ptr(), _stream())
    return out


def gemm_qkv_fused_ok(x, wqkv, qkv_out, head_dim, rotary_dim, position) -> bool:
    """Whether the q/k/v product of this step can also do the per-head norm, the rotation and the
    cache write in its epilogue: bfloat16, heads of 128 rotated whole, a step of 512 rows and more."""
    a = x.xw if isinstance(x, PendingNorm) else x
    return (options.qkv_epilogue and a.dtype == torch.bfloat16 and qkv_out.dtype == torch.bfloat16 and head_dim == 128
            and rotary_dim == 128 and position is not None and _tcgen05_ok(a, wqkv) and qkv_out.stride(0) % 8 == 0
            and qkv_out.data_ptr() % 16 == 0 and bool(_fn("hb_gemm_tcgen05_qkv_ok")(a.shape[0], wqkv.shape[0])))


def gemm_qkv_fused(x, wqkv, qkv_out, q_weight, k_weight, eps, cos, sin, tok_seq, tok_pos, seq_pages, k_cache, v_cache,
                   num_heads, num_kv_heads, page_size, write_cache, scratch) -> None:
    """qkv_out[:, :num_heads*128] = rotated (and normed) q of x @ wqkv.T; k (normed, rotated) and v go
    into the paged cache.  `x` may be a PendingNorm (its norm is finished inside)."""
    pend = x if isinstance(x, PendingNorm) else None
    a = pend.xw if pend is not None else x
    _tcgen05_workspace(qkv_out.device)
    _run("hb_gemm_tcgen05_qkv_bf16", a.data_ptr(), a.stride(0), wqkv.data_ptr(), wqkv.stride(0), qkv_out.data_ptr(), qkv_out.stride(0),
         a.shape[0], wqkv.shape[0], a.shape[1],
         pend.sumsq.data_ptr() if pend is not None else None, pend.parts if pend is not None else 0,
         pend.stride if pend is not None else 0, float(pend.eps) if pend is not None else 0.0,
         _ptr(q_weight), _ptr(k_weight), float(eps), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
         tok_seq.data_ptr(), tok_pos.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         num_heads, num_kv_heads, page_size, 1 if write_cache else 0, _error_flag(qkv_out.device).data_ptr(), _stream())


def _stream_buffers(device):
    """Per device: scratch for the K slices' partial tiles and the tiles' arrival counters (zero
    between launches).  Fixed addresses, so captured graphs can use them."""
    key = device_key(device)
    if key not in _stream_bufs:
        # K is cut into slices only while (tiles x slices) fits two CTAs per SM: that many partial tiles of 64 x 128 floats
        _stream_bufs[key] = (torch.empty(2 * sm_count(device) * 64 * 128, dtype=torch.float32, device=device),
                             torch.zeros(STREAM_COUNTERS, dtype=torch.int32, device=device))
    return _stream_bufs[key]


def gemm_stream(a, w, c, epilogue=EPI_STORE) -> None:
    """c (op)= a @ w.T for at most 64 rows of a (bfloat16): weights streamed once through TMA into
    tcgen05 tensor cores, K cut into slices that the last-arriving CTA of a tile sums in order."""
    _check(a, torch.bfloat16, "a"); _check(w, torch.bfloat16, "w"); _check(c, None, "c")
    scratch, counters = _stream_buffers(a.device)
    if w.shape[0] > STREAM_COUNTERS * 128:
        raise BackendError(f"gemm_stream: {w.shape[0]} weight rows exceed the {STREAM_COUNTERS * 128} the counters cover")
    _run("hb_gemm_stream_bf16", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), c.stride(0),
         a.shape[0], w.shape[0], a.shape[1], epilogue, scratch.data_ptr(), scratch.numel(), counters.data_ptr(),
         counters.numel(), _error_flag(a.device).data_ptr(), _stream())


def _tcgen05_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _decode_gemm(a, w):
    """Which kernel multiplies at most 64 activation rows.  Measured (microseconds at 17 / 32 / 64
    rows; mma.sync kernel, streaming tcgen05 kernel, prefill kernel) at Qwen3-8B shapes: q/k/v
    19 / 21 / 31, 23 / 23 / 28, 14 / 15 / 16; o 12 / 12 / 18, 27 / 30 / 42, 13 / 14 / 14; gate/up
    58 / 65 / 93, 46 / 49 / 57, 41 / 41 / 42; down 28 / 29 / 42, 53 / 59 / 76, 26 / 26 / 26; at 32B shapes
    the prefill kernel wins all four from 32 rows on, at 0.6B shapes (at most 6 M elements) the
    mma.sync kernel wins all four.
    Up to 16 rows the mma.sync kernel streams the weights at the memory's rate; beyond that every CTA
    of 16 weight rows reads the whole activation matrix again, and the prefill kernel (K cut over a
    cluster of CTAs where the matrix has few tiles) wins wherever the matrix is large enough to pay
    for its start and end.  The streaming kernel keeps the head."""
    if options.decode_gemm == "stream":
        return gemm_stream
    M, N, K = a.shape[0], w.shape[0], a.shape[1]
    if options.decode_gemm == "auto" and M > 16:
        elements = N * K
        if N >= 65536:
            return gemm_stream
        if _tcgen05_ok(a, w) and elements >= 16 * 1024 * 1024 and (M > 32 or N >= 6144 or elements >= 48 * 1024 * 1024):
            return gemm_tcgen05
    return gemm_skinny


def _skinny_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


# ---------------------------------------------------------------------------------------------
def _plain_input(a, scratch):
    if isinstance(a, PendingNorm):
        h = scratch(a.xw.shape, torch.bfloat16)
        finish_norm(a, h)
        return h
    return a


def gemm(a, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPI_STORE, next_norm=None, scratch=None):
    """c (op)= a @ w.T with the kernel that fits dtype and sizes.

    a [M, K] and w [N, K] share a dtype (float32: the true 32-bit product on the CUDA cores;
    bfloat16: tensor-core kernels where their size rules hold, else the any-shape kernel).
    `a` may be a PendingNorm; next_norm = (weight, eps) asks for the PendingNorm of the updated c
    (EPI_RESIDUAL), which is returned where the kernel can make it and None otherwise.
    """
    x = a.xw if isinstance(a, PendingNorm) else a
    if (isinstance(a, PendingNorm) or next_norm is not None) and scratch is not None \
            and shared_norm_ok(x.shape[0], x.dtype, w.shape[0] if next_norm is not None else 8):
        if x.shape[0] <= SHARED_NORM_MAX_ROWS and _skinny_ok(x, w):
            return gemm_skinny_norm(a, w, c, epilogue, next_norm, scratch)
        if (x.shape[0] > SKINNY_MAX_ROWS or (_skinny_ok(x, w) and _decode_gemm(x, w) is gemm_tcgen05)) \
                and _tcgen05_ok(x, w) and (next_norm is None or next_norm[0].data_ptr() % 16 == 0):
            return gemm_tcgen05_norm(a, w, c, epilogue, next_norm, scratch)
    a = _plain_input(a, scratch)
    if _skinny_ok(a, w):
        _decode_gemm(a, w)(a, w, c, epilogue)
    elif _tcgen05_ok(a, w):
        gemm_tcgen05(a, w, c, epilogue)
    else:
        gemm_simt(a, w, c, epilogue)


def gemm_swiglu(a, wgu: torch.Tensor, out: torch.Tensor, interleave: int, scratch) -> None:
    """out = silu(gate) * up with [gate | up] = a @ wgu.T.  Fused into the product where a kernel can;
    otherwise the product goes to `scratch(shape, dtype)` and the SwiGLU kernel follows."""
    if isinstance(a, PendingNorm):
        if interleave == 8 and _skinny_ok(a.xw, wgu) and a.xw.shape[0] <= SHARED_NORM_MAX_ROWS:
            gemm_skinny_norm(a, wgu, out, EPI_SWIGLU)
            return
        if interleave == 8 and _tcgen05_ok(a.xw, wgu) and \
                (a.xw.shape[0] > SKINNY_MAX_ROWS or (_skinny_ok(a.xw, wgu) and _decode_gemm(a.xw, wgu) is gemm_tcgen05)):
            gemm_tcgen05_norm(a, wgu, out, EPI_SWIGLU)
            return
        a = _plain_input(a, scratch)
    if interleave == 8 and _skinny_ok(a, wgu):
        _decode_gemm(a, wgu)(a, wgu, out, EPI_SWIGLU)
        return
    if interleave == 8 and _tcgen05_ok(a, wgu):
        gemm_tcgen05(a, wgu, out, EPI_SWIGLU)
        return
    gu = scratch((a.shape[0], wgu.shape[0]), a.dtype)
    gemm(a, wgu, gu)
    swiglu(gu, out, interleave)


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = device_key(dev)
    if key not in _sm_counts:
        _sm_counts[key] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return _sm_counts[key]


def attention_decode_scratch_floats(n_seqs, num_heads, head_dim, nsplit) -> int:
    return n_seqs * num_heads * nsplit * (head_dim + 2)


def decode_splits(n_seqs: int, num_kv_heads: int, max_tiles: int, device=None) -> int:
    """How many key ranges each (sequence, kv head) is cut into, so that the grid fills the GPU:
    `options.decode_ctas_per_sm` CTAs on every SM, one wave."""
    target = options.decode_ctas_per_sm * sm_count(device)
    want = target // max(1, n_seqs * num_kv_heads)      # rounded down: all CTAs resident at once
    # at most 16: beyond that the partial results and their combination cost more than the shorter key
    # ranges save (one sequence of 2,050 keys, 8 kv heads: 11.4 us with 16 splits, 14.8 with 37)
    return max(1, min(want, max_tiles, options.decode_max_splits))


def attention_decode(q, ldq, out, k_cache, v_cache, seq_len, seq_pages, scratch, num_heads, num_kv_heads,
                     head_dim, page_size, nsplit, scale, window, softcap=None, sink=None, gate_bias=None, out_gate=None) -> None:
    """One query per sequence (row b of q) over the cache; scratch holds the splits' partial results.
    softcap, sink and gate_bias as in `attention`; the sink joins the denominator where the splits are combined."""
    if sink is not None:
        _check(sink, torch.float32, "sink")
    if gate_bias is not None:
        _check(gate_bias, torch.float32, "gate_bias")
    _check(out, torch.bfloat16, "out"); _check(scratch, torch.float32, "scratch")
    n = out.shape[0]
    if scratch.numel() < attention_decode_scratch_floats(n, num_heads, head_dim, nsplit):
        raise BackendError("attention_decode: scratch is too small")
    _run("hb_attention_decode_bf16", q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0), k_cache.data_ptr(),
         v_cache.data_ptr(), seq_len.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0), scratch.data_ptr(),
         n, num_heads, num_kv_heads, head_dim, page_size, int(nsplit), float(scale), int(window or 0),
         float(softcap or 0.0), _ptr(sink), _ptr(gate_bias), *_out_gate(out_gate, n, num_heads), _stream())


_DECODE_COUNTERS = 65536
_decode_counters: dict = {}


def attention_decode_fused_ok(qkv, out, num_heads, num_kv_heads, head_dim, page_size, rotary_dim, n_seqs) -> bool:
    """Whether one launch can do norm, rotation, cache write, attention and combine for this step."""
    return (options.decode_fused and out.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16
            and head_dim == 128 and rotary_dim == head_dim and num_heads // num_kv_heads <= 16 and page_size % 64 == 0
            and qkv.stride(0) % 4 == 0 and qkv.data_ptr() % 8 == 0 and n_seqs * num_kv_heads <= _DECODE_COUNTERS)


def attention_decode_fused(qkv, out, k_cache, v_cache, q_weight, k_weight, eps, cos, sin, write_cache, seq_len,
                           seq_pages, scratch, num_heads, num_kv_heads, page_size, nsplit, scale, window) -> None:
    """Head size 128: the new token's q and k get their per-head norm and rotation, k and v go into
    the cache, every query attends its sequence's keys, and the key splits are combined: one kernel."""
    _check(out, torch.bfloat16, "out"); _check(scratch, torch.float32, "scratch"); _check(qkv, torch.bfloat16, "qkv")
    n = out.shape[0]
    if scratch.numel() < attention_decode_scratch_floats(n, num_heads, 128, nsplit):
        raise BackendError("attention_decode_fused: scratch is too small")
    key = device_key(out.device)
    if key not in _decode_counters:
        _decode_counters[key] = torch.zeros(_DECODE_COUNTERS, dtype=torch.int32, device=out.device)
    _run("hb_attention_decode_fused_bf16", qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), _ptr(q_weight), _ptr(k_weight), float(eps), cos.data_ptr(), sin.data_ptr(),
         cos.shape[0], 1 if write_cache else 0, seq_len.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
         scratch.data_ptr(), _decode_counters[key].data_ptr(), n, num_heads, num_kv_heads, page_size, int(nsplit),
         float(scale), int(window or 0), _stream())


def attention_prefill(q, ldq, out, k_cache, v_cache, seq_start, seq_pos0, seq_pages, n_seqs, max_q_len,
                      num_heads, num_kv_heads, head_dim, page_size, scale, window, softcap=None, sink=None,
                      gate_bias=None, out_gate=None) -> None:
    """Causal attention of packed query rows (seq_start marks the sequences) over the cache."""
    _check(out, torch.bfloat16, "out")
    if sink is not None:
        _check(sink, torch.float32, "sink")
    if gate_bias is not None:
        _check(gate_bias, torch.float32, "gate_bias")
    _run("hb_attention_prefill_bf16", q.data_ptr(), int(ldq), out.data_ptr(), out.stride(0), k_cache.data_ptr(),
         v_cache.data_ptr(), seq_start.data_ptr(), seq_pos0.data_ptr(), seq_pages.data_ptr(), seq_pages.stride(0),
         int(n_seqs), int(max_q_len), num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
         float(softcap or 0.0), _ptr(sink), _ptr(gate_bias), *_out_gate(out_gate, out.shape[0], num_heads), _stream())


def attention_prefill_tc(q, ldq, out, k_cache, v_cache, seq_start, seq_pos0, seq_pages, n_seqs, max_q_len,
                         num_heads, num_kv_heads, head_dim, page_size, scale, window, softcap=None, sink=None,
                         gate_bias=None, out_gate=None) -> None:
    """The same on tcgen05 tensor cores (head sizes 64 and 128): S and O in tensor memory."""
    _check(out, torch.bfloat16, "out")
    if sink is not None:
        _check(sink, torch.float32, "sink")
    if gate_bias is not None:
        _check(gate_bias, torch.float32, "gate_bias")
    _run("hb_attention_prefill_tc_bf16", q.data_ptr(), int(ldq), q.shape[0], out.data_ptr(), out.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0], seq_start.data_ptr(), seq_pos0.data_ptr(),
         seq_pages.data_ptr(), seq_pages.stride(0), int(n_seqs), int(max_q_len), num_heads, num_kv_heads, head_dim,
         page_size, float(scale), int(window or 0), float(softcap or 0.0), _ptr(sink), _ptr(gate_bias),
         *_out_gate(out_gate, out.shape[0], num_heads), _error_flag(out.device).data_ptr(), _work_counter(out.device).data_ptr(),
         _stream())


_work_counters: dict = {}


def _work_counter(device) -> torch.Tensor:
    """One int per device from which the CTAs of a persistent kernel take their next item of work;
    zero between launches (the CTA that fetches last puts it back)."""
    key = device_key(device)
    if key not in _work_counters:
        _work_counters[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _work_counters[key]


def _prefill_tc_ok(q, ldq, out, head_dim, page_size) -> bool:
    return (options.prefill_attention == "tcgen05" and out.dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 64 == 0
            and ldq % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def _prefill_kernel_ok(out, head_dim, page_size) -> bool:
    return out.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and page_size % 64 == 0


def _decode_kernel_ok(out, num_heads, num_kv_heads, head_dim, page_size) -> bool:
    return (out.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and num_heads // num_kv_heads <= 16 and page_size % 64 == 0)


def attention(q, ldq, out, k_cache, v_cache, batch, num_heads, num_kv_heads, head_dim, page_size,
              scale, window, seq_pages, scratch=None, softcap=None, sink=None, gate_bias=None, out_gate=None) -> None:
    """Attention of every token of the step over its sequence's cached keys and values.

    bfloat16 steps of one token per sequence take the split-key tensor-core kernel, other bfloat16
    steps the flash kernel; head sizes or pages those cannot serve, and the float32 path, take
    the any-shape kernel.  Every kernel takes a cap on the scores (softcap c: s <- c * tanh(s / c)) and a sink
    (a float per query head whose exponential joins the softmax's denominator); v_cache may be k_cache.  With
    `gate_bias` (a float per query head) there is no softmax: a visible key weighs sigmoid(score + gate_bias[head]).  With
    `out_gate` (float [tokens, num_heads]) a head's result is multiplied by sigmoid(out_gate[token, head]) before it is rounded."""
    if options.attention == "simt":
        attention_simt(q, ldq, out, k_cache, v_cache, batch.tok_seq, batch.tok_pos, seq_pages, num_heads,
                       num_kv_heads, head_dim, page_size, scale, window, softcap, sink, gate_bias, out_gate)
        return
    if batch.is_decode and scratch is not None and _decode_kernel_ok(out, num_heads, num_kv_heads, head_dim, page_size):
        tiles = seq_pages.shape[1] * (page_size // 64)
        nsplit = decode_splits(batch.n_seqs, num_kv_heads, tiles)
        buf = scratch((attention_decode_scratch_floats(batch.n_seqs, num_heads, head_dim, nsplit),), torch.float32)
        attention_decode(q, ldq, out, k_cache, v_cache, batch.seq_len, seq_pages, buf, num_heads, num_kv_heads,
                         head_dim, page_size, nsplit, scale, window, softcap, sink, gate_bias, out_gate)
        return
    if _prefill_tc_ok(q, ldq, out, head_dim, page_size):
        attention_prefill_tc(q, ldq, out, k_cache, v_cache, batch.seq_start, batch.seq_pos0, seq_pages, batch.n_seqs,
                             batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size, scale, window, softcap, sink, gate_bias,
                             out_gate)
        return
    if _prefill_kernel_ok(out, head_dim, page_size):
        attention_prefill(q, ldq, out, k_cache, v_cache, batch.seq_start, batch.seq_pos0, seq_pages, batch.n_seqs,
                          batch.max_q_len, num_heads, num_kv_heads, head_dim, page_size, scale, window, softcap, sink, gate_bias,
                          out_gate)
        return
    attention_simt(q, ldq, out, k_cache, v_cache, batch.tok_seq, batch.tok_pos, seq_pages, num_heads,
                   num_kv_heads, head_dim, page_size, scale, window, softcap, sink, gate_bias, out_gate)
