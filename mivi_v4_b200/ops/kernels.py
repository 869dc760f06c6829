"""Launch wrappers: one Python function per kernel entry point.

Every wrapper checks what the kernel assumes (device, dtype, contiguity,
shapes, size limits) and raises ``KernelError`` with the offending value
instead of launching; the kernels themselves check nothing.  There is no CPU
implementation behind these functions: a tensor that is not on a CUDA device
is an error, and so is a library that cannot be built.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .build import DEBUG_CHECKS, load_library

F32, BF16 = 0, 1
MAX_HEAD_DIM = 256
MAX_CONV_K = 16
RECENT_MAX = 64
RECENT_RING = 128


class KernelError(RuntimeError):
    pass


_P, _I, _F, _Q, _UQ = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong
_SIGNATURES = {
    "core": {
        "mv_embed": [_P, _I, _P, _P, _I, _I, _P],
        "mv_embed_link": [_P, _I, _P, _P, _I, _I, _P, _P, _P, _I, _P],
        "mv_embed_link_partials": [_I],
        "mv_rmsnorm": [_P, _P, _P, _I, _P, _I, _I, _F, _P],
        "mv_swiglu": [_P, _P, _I, _I, _I, _I, _P],
        "mv_copy_to_host": [_P, _P, _Q, _P],
        "mv_delay": [_Q, _P],
        "mv_gemm_simt": [_P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_shortconv_decode": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "mv_qk_prepare": [_P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _Q, _I, _P, _I, _I, _I, _I, _I, _P],
        "mv_attention_generic": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
        "mv_attention_decode": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I,
                                _I, _I, _P],
        "mv_layernorm": [_P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
        "mv_gated_rmsnorm": [_P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _F, _I, _P],
        "mv_rmsnorm_add": [_P, _P, _P, _I, _I, _F, _P],
        "mv_rmsnorm_add_layernorm": [_P, _P, _F, _P, _P, _F, _P, _I, _I, _I, _P],
        "mv_glu_clamped": [_P, _P, _I, _I, _I, _F, _F, _P],
        "mv_table_gate": [_P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _P],
        "mv_table_gate_proj": [_P, _P, _P, _I, _I, _I, _P, _P, _I, _I, _I, _P],
        "mv_round_rows": [_P, _P, _I, _Q, _P],
        "mv_decay_scan": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _F, _F, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "mv_decay_chunks": [_I, _I],
        "mv_decay_scan_chunked": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _F, _F, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I,
                                  _I, _I, _I, _P],
        "mv_qkv_prepare_wide": [_P, _I, _P, _P, _F, _I, _P, _P, _P, _P, _I, _I, _P, _Q, _P, _I, _I, _I, _I, _I, _I, _I,
                                _F, _P],
        "mv_attention_sink": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I,
                              _I, _I, _P, _P, _I, _I, _P, _P],
        "mv_mix_heads": [_P, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_block_gates": [_P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P],
        "mv_gated_recurrence": [_P, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _P],
        "mv_scaled_add_norm": [_P, _F, _P, _F, _P, _P, _P, _F, _P, _I, _I, _I, _P],
        "mv_embed_scaled_pos": [_P, _I, _P, _F, _P, _P, _P, _P, _I, _I, _I, _P],
        "mv_softcap": [_P, _Q, _F, _P],
        "mv_rmsnorm_add_sum": [_P, _F, _P, _F, _P, _P, _P, _I, _I, _I, _F, _P],
        "mv_scalar_scan": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I,
                           _P],
        "mv_scalar_chunks": [_I, _I],
        "mv_scalar_scan_chunked": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _F, _P, _P, _P, _P, _P, _P, _I, _I, _I,
                                   _I, _I, _I, _I, _I, _P],
        "mv_memory_gates": [_P, _I, _P, _I, _P, _P, _F, _P, _P, _P, _P, _P, _P, _I, _I, _P],
        "mv_causal_conv": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "mv_ssm_decode_prepare": [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P, _I, _P, _P, _P, _P, _I, _P],
        "mv_step_size": [_P, _I, _P, _P, _P, _P, _I, _I, _P],
        "mv_route": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _F, _I, _P],
        "mv_routed_glu": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
        "mv_scale_expert_columns": [_P, _I, _P, _I, _I, _I, _I, _I, _P],
        "mv_identity_experts": [_P, _I, _P, _I, _I, _I, _P, _I, _I, _I, _P],
        "mv_embed_bigram": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _Q, _Q, _P],
        "mv_add_rows_vector": [_P, _P, _P, _I, _I, _P],
        "mv_latent_prepare": [_P, _I, _I, _I, _P, _F, _P, _P, _P, _P, _I, _I, _P, _Q, _I, _P, _I, _I, _I, _I, _I, _I, _P],
        "mv_head_product": [_P, _Q, _I, _P, _I, _I, _P, _Q, _P, _I, _Q, _I, _I, _I, _I, _I, _P],
        "mv_latent_attention": [_P, _P, _Q, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _P, _P, _P],
        "mv_delta_scan_long": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _F, _F, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
        "mv_delta_scan": [_P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _F, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
        "mv_expert_rank": [_P, _I, _I, _P, _P, _P],
        "mv_expert_gather": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P],
        "mv_expert_tiles": [_P, _I, _I, _P, _P, _I, _P],
        "mv_expert_combine": [_P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P],
        "mv_sample": [_P, _Q, _P, _I, _I, _F, _I, _F, _F, _F, _F, _F, _P, _P, _UQ, _P, _P, _P, _P, _P, _P, _P, _P],
    },
    "bf16": {
        "mv_gemm_small_m": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _Q, _P],
        "mv_gemm_small_m_tile_rows": [_I, _I],
        "mv_gemm_small_m_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _Q, _P],
        "mv_gemm_small_m_heads": [_P, _P, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _P, _Q, _P, _I, _I, _I, _I,
                                  _P, _I, _I, _I, _F, _P, _Q, _P],
        "mv_gemm_tc": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P],
        "mv_gemm_tc_grouped": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P],
        "mv_gemm_tc_pair": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _P],
        "mv_gemm_tc_swap": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _P, _P, _I, _P, _Q, _P, _P],
        "mv_gemm_tc_swap_shortconv": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _I, _F, _P, _Q,
                                      _P, _P],
        "mv_gemm_tc_swap_heads": [_P, _P, _P, _P, _F, _P, _P, _P, _P, _I, _I, _P, _Q, _P, _I, _I, _I, _I,
                                  _P, _I, _I, _I, _F, _P, _Q, _P, _P],
        "mv_attention_prefill": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P],
        "mv_attention_sink_prefill": [_P, _P, _Q, _P, _I, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _F, _I,
                                      _I, _I, _P, _P, _I, _I, _P, _I, _P],
        "mv_attention_decode_tc": [_P, _P, _Q, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P, _P],
        "mv_attention_prefill_tc": [_P, _P, _Q, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _P, _P],
        "mv_latent_query": [_P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P],
        "mv_latent_gather": [_P, _Q, _P, _I, _I, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P],
        "mv_latent_attention_prefill": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    },
}
_fns = {}


class KernelProfile:
    """Device time of every launch made while it is active, by stage of the model and by entry point,
    with the bytes and floating-point operations that the launch's wrapper accounts for it.

    The reference times the stages of its forward pass behind a switch (embedding, attention and its
    stages, the convolution layers and their stages, logits: crates/mivi-model/src/model.rs:57-74,
    273-293) and prints them from its ``bench`` command.  Here every launch is bracketed by two CUDA
    events on the launching stream; that keeps consecutive kernels from overlapping, so the sum is a
    little more than what the same step takes when it is replayed from a recording."""

    def __init__(self):
        self.records = []            # [stage, entry point, start event, end event, bytes, flops]
        self.stage = "-"
        self.steps = 0

    def wrap(self, name: str, f):
        def timed(*args):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            code = f(*args)
            e1.record()
            self.records.append([self.stage, name, e0, e1, 0, 0])
            return code
        return timed

    def account(self, nbytes: int, flops: int) -> None:
        if self.records:
            self.records[-1][4] += int(nbytes)
            self.records[-1][5] += int(flops)

    def report(self, reset: bool = True) -> dict:
        """{"rows": [{stage, kernel, calls, us, share, gb_per_s, tflops}], "stages": {stage: us}, "total_us",
        "steps"}: rows sorted by time.  Waits for the device."""
        torch.cuda.synchronize()
        agg = {}
        for stage, name, e0, e1, nbytes, flops in self.records:
            row = agg.setdefault((stage, name), [0, 0.0, 0, 0])
            row[0] += 1
            row[1] += e0.elapsed_time(e1) * 1e3
            row[2] += nbytes
            row[3] += flops
        total = sum(r[1] for r in agg.values()) or 1.0
        rows = [dict(stage=k[0], kernel=k[1], calls=r[0], us=r[1], share=r[1] / total,
                     gb_per_s=(r[2] / r[1] / 1e3) if r[2] else None, tflops=(r[3] / r[1] / 1e6) if r[3] else None)
                for k, r in sorted(agg.items(), key=lambda kv: -kv[1][1])]
        stages = {}
        for row in rows:
            stages[row["stage"]] = stages.get(row["stage"], 0.0) + row["us"]
        out = dict(rows=rows, stages=stages, total_us=total, steps=self.steps)
        if reset:
            self.records, self.steps = [], 0
        return out


_profile: Optional[KernelProfile] = None


class _NoStage:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_STAGE = _NoStage()


class _Stage:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.prev, _profile.stage = _profile.stage, self.name

    def __exit__(self, *exc):
        if _profile is not None:
            _profile.stage = self.prev
        return False


def profile_stage(name: str):
    """``with profile_stage("mixer gqa"):`` names the stage of the launches inside, when a profile is active."""
    return _Stage(name) if _profile is not None else _NO_STAGE


class profiling:
    """``with profiling(p):`` every launch inside is timed into ``p`` (a KernelProfile, or None: nothing)."""

    def __init__(self, p: Optional[KernelProfile]):
        self.p = p

    def __enter__(self):
        global _profile
        self.prev, _profile = _profile, self.p
        return self.p

    def __exit__(self, *exc):
        global _profile
        _profile = self.prev
        return False


def delay(us: int) -> None:
    """Keep the current stream busy for ``us`` microseconds (at most 50,000)."""
    code = _fn("core", "mv_delay")(int(us), _stream())
    if code != 0:
        raise KernelError(f"mv_delay: launch failed with CUDA error {code}")


def profiling_on() -> bool:
    return _profile is not None


def account(nbytes: int = 0, flops: int = 0) -> None:
    """Bytes that the last launch has to move and operations it has to do, for the active profile."""
    if _profile is not None:
        _profile.account(nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _fn(lib: str, name: str):
    key = (lib, name)
    f = _fns.get(key)
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = _SIGNATURES[lib][name]
        f.restype = ctypes.c_int
        _fns[key] = f
    if _profile is not None and not name.endswith(("_partials", "_tile_rows", "_to_host", "_delay", "_chunks")):
        return _profile.wrap(name, f)
    return f


def _guard(lib: str, file: str, device, n_pages: int = 0x7fffffff, n_slots: int = 0x7fffffff) -> None:
    """In a build with index checks: declare, for the kernels of one source file, how many pages and slots
    the tensors of the next launch really have.  Nothing in an ordinary build."""
    if not DEBUG_CHECKS:
        return
    name = "mv_set_guard_" + file
    f = _fns.get((lib, name))
    if f is None:
        f = getattr(load_library(lib), name)
        f.argtypes = [_I, _I, _P, _P]
        f.restype = ctypes.c_int
        _fns[(lib, name)] = f
    code = f(int(min(n_pages, 0x7fffffff)), int(min(n_slots, 0x7fffffff)), _error_flag(device).data_ptr(), _stream())
    if code != 0:
        raise KernelError(f"{name}: CUDA error {code}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  A step asks a hundred times: the two direct calls cost a
    tenth of building a ``torch.cuda.Stream`` object each time."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16")


def _need(t: Optional[torch.Tensor], name: str, dtype=None, shape=None, optional=False):
    if t is None:
        if optional:
            return None
        raise KernelError(f"{name}: missing tensor")
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; this library runs on CUDA devices only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor is not contiguous (strides {t.stride()})")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        have = t.shape
        bad = len(shape) != len(have)
        if not bad:
            for s, d in zip(shape, have):         # a plain loop: this runs hundreds of times a step
                if s is not None and s != d:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{name}: shape {tuple(have)}, expected {tuple(shape)}")
    return t.data_ptr()


_launches = 0
# kernels launched by one call of each entry point
_KERNELS_PER_CALL = {"mv_shortconv": 2, "mv_decay_scan_chunked": 2, "mv_causal_conv": 2, "mv_scalar_scan_chunked": 2}


def launch_count() -> int:
    """Kernels of this library launched so far in this process."""
    return _launches


def add_launches(n: int) -> None:
    """Kernels that ran without passing through a wrapper (a replayed CUDA graph)."""
    global _launches
    _launches += n


def _check(code: int, name: str) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{name}: launch failed with CUDA error {code}")
    _launches += _KERNELS_PER_CALL.get(name, 1)


# --------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor,
          emit: Optional["NormLink"] = None) -> torch.Tensor:
    """out[n, :] = table[tokens[n], :] widened to float32.  ``emit``: a :class:`NormLink` whose rows
    bf16(out * weight) and partial sums of squares the kernel writes too, for the product after it."""
    N = tokens.numel()
    V, H = table.shape
    if emit is not None:
        n_part = int(_fn("core", "mv_embed_link_partials")(H))
        _need(emit.partials, "norm partials", torch.float32)
        if emit.dim != H or emit.partials.dim() != 2 or emit.partials.shape[0] < N or emit.partials.shape[1] < n_part:
            raise KernelError(f"embed: a norm link of width {emit.dim} with partials "
                              f"{tuple(emit.partials.shape)} cannot take {N} rows of {H}")
        _check(_fn("core", "mv_embed_link")(
            _need(table, "embedding table"), _dt(table), _need(tokens, "tokens", torch.int32),
            _need(out, "embedding out", torch.float32, (N, H)), N, H,
            _need(emit.weight, "norm weight", torch.float32, (H,)),
            _need(emit.xg, "normed rows", torch.bfloat16, (N, H)), emit.partials.data_ptr(), emit.partials.shape[1],
            _stream()), "mv_embed_link")
        emit.n_partials = n_part
        account(N * H * (table.element_size() + 4 + 2))
        return out
    _check(_fn("core", "mv_embed")(
        _need(table, "embedding table"), _dt(table), _need(tokens, "tokens", torch.int32),
        _need(out, "embedding out", torch.float32, (N, H)), N, H, _stream()), "mv_embed")
    account(N * H * (table.element_size() + 4))
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rmsnorm(x[rows[i]] or x[i]) * w, statistics in float32."""
    H = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    _check(_fn("core", "mv_rmsnorm")(
        _need(x, "rmsnorm x", torch.float32), _need(w, "rmsnorm weight", torch.float32, (H,)),
        _need(out, "rmsnorm out", None, (n, H)), _dt(out),
        _need(rows, "rmsnorm rows", torch.int32, optional=True), n, H, float(eps), _stream()), "mv_rmsnorm")
    account(n * H * (4 + out.element_size()))
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = (x[r] - mean) / sqrt(var + eps) * w (+ bias) with r = rows[i] or i; statistics in float32,
    the variance being the mean of the squared deviations."""
    H = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    _check(_fn("core", "mv_layernorm")(
        _need(x, "layernorm x", torch.float32), _need(w, "layernorm weight", torch.float32, (H,)),
        _need(bias, "layernorm bias", torch.float32, (H,), True), _need(out, "layernorm out", None, (n, H)), _dt(out),
        _need(rows, "layernorm rows", torch.int32, optional=True), n, H, float(eps), _stream()), "mv_layernorm")
    account(n * H * (4 + out.element_size()))
    return out


GATE_SILU, GATE_SIGMOID, GATE_SILU_FIRST = 0, 1, 2


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group: int, eps: float, act: int,
                  out: torch.Tensor) -> torch.Tensor:
    """Every group of ``group`` consecutive values of a row of x [N, C] (float32) is divided by its root mean
    square, multiplied by w[c mod len(w)] and by act(gate[n, c]): ``GATE_SILU`` or ``GATE_SIGMOID``.  With
    ``GATE_SILU_FIRST`` the gate comes before the norm: x * silu(gate) is divided by ITS root mean square and
    multiplied by w.  ``gate`` (float32) may be a column slice of a wider matrix: only its rows must be contiguous."""
    N, C = x.shape
    if group < 1 or C % group:
        raise KernelError(f"gated_rmsnorm: rows of {C} values do not split into groups of {group}")
    if w.numel() not in (group, C):
        raise KernelError(f"gated_rmsnorm: {w.numel()} weights for groups of {group} in rows of {C}")
    if (not gate.is_cuda or gate.dtype != torch.float32 or gate.dim() != 2 or tuple(gate.shape) != (N, C)
            or gate.stride(1) != 1):
        raise KernelError(f"gated_rmsnorm: gate must be float32 [{N}, {C}] with unit column stride, got "
                          f"{gate.dtype} {tuple(gate.shape)} strides {gate.stride()}")
    _check(_fn("core", "mv_gated_rmsnorm")(
        _need(x, "gated_rmsnorm x", torch.float32), gate.data_ptr(), gate.stride(0),
        _need(w, "gated_rmsnorm weight", torch.float32), w.numel(), _need(out, "gated_rmsnorm out", None, (N, C)),
        _dt(out), N, C, int(group), float(eps), int(act), _stream()), "mv_gated_rmsnorm")
    account(N * C * (8 + out.element_size()))
    return out


def rmsnorm_add(y: torch.Tensor, w: torch.Tensor, eps: float, resid: torch.Tensor) -> torch.Tensor:
    """resid += y / sqrt(mean(y^2) + eps) * w, row by row, all float32."""
    N, H = y.shape
    _check(_fn("core", "mv_rmsnorm_add")(
        _need(y, "rmsnorm_add y", torch.float32), _need(w, "rmsnorm_add weight", torch.float32, (H,)),
        _need(resid, "residual stream", torch.float32, (N, H)), N, H, float(eps), _stream()), "mv_rmsnorm_add")
    account(N * H * 12)
    return resid


def rmsnorm_add_layernorm(y: torch.Tensor, w: torch.Tensor, eps: float, resid: torch.Tensor, ln_w: torch.Tensor,
                          ln_eps: float, out: torch.Tensor) -> torch.Tensor:
    """``rmsnorm_add`` followed by ``layernorm`` of the rows it has completed, in one kernel: resid += y / rms(y) * w,
    out = layer_norm(resid) * ln_w (no bias)."""
    N, H = y.shape
    _check(_fn("core", "mv_rmsnorm_add_layernorm")(
        _need(y, "rmsnorm_add y", torch.float32), _need(w, "rmsnorm_add weight", torch.float32, (H,)), float(eps),
        _need(resid, "residual stream", torch.float32, (N, H)), _need(ln_w, "layernorm weight", torch.float32, (H,)),
        float(ln_eps), _need(out, "layernorm out", None, (N, H)), _dt(out), N, H, _stream()), "mv_rmsnorm_add_layernorm")
    account(N * H * (12 + out.element_size()))
    return out


def glu_clamped(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate and
    up are the two halves of a row of ``gu`` (float32)."""
    N, F2 = gu.shape
    F = F2 // 2
    _check(_fn("core", "mv_glu_clamped")(
        _need(gu, "glu in", torch.float32, (N, 2 * F)), _need(out, "glu out", None, (N, F)), _dt(out), N, F,
        float(limit), float(alpha), _stream()), "mv_glu_clamped")
    account(_nbytes(gu, out))
    return out


def table_gate(p: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, d] = gelu_tanh(p[n, d]) * table[tokens[n], col0 + d]: a projection gated by a slice of a
    per-token table row."""
    N, D = p.shape
    if table.dim() != 2 or col0 < 0 or col0 + D > table.shape[1]:
        raise KernelError(f"table_gate: columns {col0}..{col0 + D} are outside a table of {tuple(table.shape)}")
    if _dt(table) == BF16 and _dt(out) != BF16:
        raise KernelError("table_gate: a bfloat16 table needs a bfloat16 output")
    _check(_fn("core", "mv_table_gate")(
        _need(p, "table_gate p", torch.float32), _need(table, "table_gate table"), _dt(table), table.shape[1],
        int(col0), _need(tokens, "tokens", torch.int32), _need(out, "table_gate out", None, (N, D)), _dt(out), N, D,
        _stream()), "mv_table_gate")
    account(_nbytes(p, out) + N * D * table.element_size())
    return out


TABLE_GATE_PROJ_MAX_ROWS = 64


def table_gate_proj_ok(n_rows: int, gate: torch.Tensor, table: torch.Tensor, dtype: torch.dtype) -> bool:
    """Whether ``table_gate_proj`` takes a step: few rows (every token re-reads the matrix), matrix and table in
    the run's dtype."""
    return 1 <= n_rows <= TABLE_GATE_PROJ_MAX_ROWS and gate.dtype == table.dtype == dtype


def table_gate_proj(resid: torch.Tensor, gate: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor,
                    out: torch.Tensor) -> torch.Tensor:
    """out[n, d] = gelu_tanh(gate[d] . x_n) * table[tokens[n], col0 + d], x_n being row n of ``resid`` (float32)
    rounded to the matrix's dtype: ``round_rows``, a product and ``table_gate`` in one kernel, for few rows."""
    N, H = resid.shape
    D = gate.shape[0]
    if not table_gate_proj_ok(N, gate, table, out.dtype):
        raise KernelError("table_gate_proj: too many rows or mixed dtypes; ask table_gate_proj_ok first")
    if gate.shape[1] != H or col0 < 0 or col0 + D > table.shape[1]:
        raise KernelError(f"table_gate_proj: gate {tuple(gate.shape)} and columns {col0}..{col0 + D} of a table "
                          f"{tuple(table.shape)} do not fit rows of {H}")
    _check(_fn("core", "mv_table_gate_proj")(
        _need(resid, "residual stream", torch.float32), _need(gate, "gate matrix"), _need(table, "table"), _dt(gate),
        table.shape[1], int(col0), _need(tokens, "tokens", torch.int32), _need(out, "table_gate_proj out", None, (N, D)),
        N, H, D, _stream()), "mv_table_gate_proj")
    account(N * (H * D * gate.element_size() + 4 * H), 2 * N * H * D)
    return out


def round_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = x (float32) rounded to out's dtype."""
    _check(_fn("core", "mv_round_rows")(
        _need(x, "round_rows x", torch.float32), _need(out, "round_rows out", None, tuple(x.shape)), _dt(out),
        x.numel(), _stream()), "mv_round_rows")
    account(_nbytes(x, out))
    return out


def embed_scaled_pos(table: torch.Tensor, tokens: torch.Tensor, scale: float, pos_table: Optional[torch.Tensor],
                     positions: torch.Tensor, out: torch.Tensor, rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[n] = table[tokens[n]] * scale + pos_table[positions[n]] in float32 (``pos_table`` None: no position
    vector); ``rounded`` also gets the rows in its own dtype."""
    N, H = out.shape
    if pos_table is not None and pos_table.dtype != table.dtype:
        raise KernelError(f"embed: the token table is {table.dtype}, the position table {pos_table.dtype}")
    _check(_fn("core", "mv_embed_scaled_pos")(
        _need(table, "embedding table", None, (None, H)), _dt(table), _need(tokens, "tokens", torch.int32), float(scale),
        _need(pos_table, "position table", None, (None, H), True), _need(positions, "positions", torch.int32),
        _need(out, "embed out", torch.float32), _need(rounded, "embed rounded", None, (N, H), True),
        _dt(rounded) if rounded is not None else F32, N, H, _stream()), "mv_embed_scaled_pos")
    account(N * H * (2 * table.element_size() + 4))
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _check(_fn("core", "mv_softcap")(_need(x, "softcap x", torch.float32), x.numel(), float(cap), _stream()), "mv_softcap")
    account(x.numel() * 8)
    return x


def rmsnorm_add_sum(y1: torch.Tensor, w: torch.Tensor, eps: float, resid: torch.Tensor, *, s1: float = 1.0,
                    y2: Optional[torch.Tensor] = None, s2: float = 1.0, rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid += y / sqrt(mean(y^2) + eps) * w with y = s1 * y1 (+ s2 * y2), all float32; ``rounded`` also gets
    the completed rows in its own dtype (what the next sublayer multiplies)."""
    N, H = y1.shape
    _check(_fn("core", "mv_rmsnorm_add_sum")(
        _need(y1, "rmsnorm_add_sum y1", torch.float32), float(s1), _need(y2, "rmsnorm_add_sum y2", torch.float32, (N, H), True),
        float(s2), _need(w, "rmsnorm_add_sum weight", torch.float32, (H,)),
        _need(resid, "residual stream", torch.float32, (N, H)), _need(rounded, "rounded rows", None, (N, H), True),
        _dt(rounded) if rounded is not None else F32, N, H, float(eps), _stream()), "mv_rmsnorm_add_sum")
    account(N * H * (12 + (4 if y2 is not None else 0) + (rounded.element_size() if rounded is not None else 0)))
    return resid


def scaled_add_norm(y1: torch.Tensor, vec: torch.Tensor, resid: torch.Tensor, *, s1: float = 1.0,
                    y2: Optional[torch.Tensor] = None, s2: float = 1.0, w: Optional[torch.Tensor] = None,
                    eps: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid[n, :] += vec * (s1 y1[n, :] + s2 y2[n, :]) (``y2`` None: s1 y1): a sublayer's result, or the weighted
    sum of two, times a learned vector, joins the float32 stream.  With ``w`` and ``out`` the completed row is
    normed for the next sublayer in the same kernel: out[n, :] = resid / sqrt(mean(resid^2) + eps) * w."""
    N, H = resid.shape
    if (w is None) != (out is None):
        raise KernelError("scaled_add_norm: the norm's weight and its output come together")
    _check(_fn("core", "mv_scaled_add_norm")(
        _need(y1, "scaled_add_norm y1", torch.float32, (N, H)), float(s1),
        _need(y2, "scaled_add_norm y2", torch.float32, (N, H), True), float(s2),
        _need(vec, "scaled_add_norm vector", torch.float32, (H,)), _need(resid, "resid", torch.float32),
        _need(w, "norm weight", torch.float32, (H,), True), float(eps), _need(out, "scaled_add_norm out", None, (N, H), True),
        _dt(out) if out is not None else F32, N, H, _stream()), "mv_scaled_add_norm")
    account(N * H * (12 + (4 if y2 is not None else 0) + (out.element_size() if out is not None else 0)))
    return resid


def block_gates(u: torch.Tensor, wa_t: torch.Tensor, wi_t: torch.Tensor, ba: torch.Tensor, bi: torch.Tensor,
                lam: torch.Tensor, c: float, a_out: torch.Tensor, x_out: torch.Tensor) -> None:
    """The gates of a gated linear recurrence, float32: with u [N, C] cut into ``n_blocks`` = wa_t.shape[0] equal
    parts, r = sigmoid(A_b u_b + ba), i = sigmoid(B_b u_b + bi); a_out = exp(-c r softplus(lam)) and
    x_out = sqrt(1 - a^2) i u.  ``wa_t``, ``wi_t`` [n_blocks, in, out]: the parts' square matrices TRANSPOSED."""
    N, C = u.shape
    nb = wa_t.shape[0]
    if nb < 1 or C % nb:
        raise KernelError(f"block_gates: {C} channels do not split into {nb} parts")
    bs = C // nb
    if bs * 64 > 160 * 1024:
        raise KernelError(f"block_gates: parts of {bs} channels are more than a block holds (2,560)")
    _check(_fn("core", "mv_block_gates")(
        _need(u, "block_gates input", torch.float32, (N, C)), _need(wa_t, "block_gates A", torch.float32, (nb, bs, bs)),
        _need(wi_t, "block_gates B", torch.float32, (nb, bs, bs)), _need(ba, "block_gates A bias", torch.float32, (C,)),
        _need(bi, "block_gates B bias", torch.float32, (C,)), _need(lam, "block_gates lambda", torch.float32, (C,)), float(c),
        _need(a_out, "block_gates decay out", torch.float32, (N, C)), _need(x_out, "block_gates input out", torch.float32, (N, C)),
        N, C, nb, _stream()), "mv_block_gates")
    account(N * C * 12 + 2 * nb * bs * bs * 4, 4 * N * C * bs)


def gated_recurrence(a: torch.Tensor, x: torch.Tensor, y: torch.Tensor, state: torch.Tensor, slots, cu, out: torch.Tensor,
                     n_seqs: int, max_len: int = 1) -> torch.Tensor:
    """S_t = a_t S_(t-1) + x_t per channel along each sequence, from the state kept per slot (float32 [slots, C],
    brought up to date); out = S * gelu_tanh(y) in ``out``'s dtype.  a, x float32 [N, C]; y float32 [N, C], a column
    slice is fine.  ``max_len``: the most tokens that a sequence brings; long sequences are walked in pieces."""
    N, C = out.shape
    yp, ldy = _cols(y, "gated_recurrence y", N, C)
    _guard("core", "gated_recurrence", out.device, n_slots=state.shape[0])
    _check(_fn("core", "mv_gated_recurrence")(
        _need(a, "gated_recurrence decay", torch.float32, (N, C)), _need(x, "gated_recurrence input", torch.float32, (N, C)),
        yp, ldy, _need(state, "gated_recurrence state", torch.float32, (None, C)), _need(slots, "slots", torch.int32),
        _need(cu, "cu", torch.int32), _need(out, "gated_recurrence out"), _dt(out), int(n_seqs), C, int(max_len), _stream()),
        "mv_gated_recurrence")
    account(N * C * (12 + out.element_size()) + 2 * n_seqs * C * 4, 4 * N * C)
    return out


def scalar_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, log_a: torch.Tensor, b: torch.Tensor,
                state: torch.Tensor, slots: torch.Tensor, cu: torch.Tensor, out: torch.Tensor, n_seqs: int,
                n_heads: int, dk: int, dv: int, *, heads_per_group: int = 1, skip: Optional[torch.Tensor] = None,
                m_tok: Optional[torch.Tensor] = None, q_scale: float = 1.0, max_len: int = 1, ws=None) -> torch.Tensor:
    """A matrix state per head with ONE decay per token and head: S <- a_t S + b_t k_t v_t^T, o_t = S^T q_t
    (+ skip_h v_t), over the step's tokens in order, from and into ``state`` [slots, heads, dv (+ 1), dk]
    (float32).  ``log_a`` and ``b`` [N, heads] are float32 (column slices are fine); q, k [N, groups * dk]
    with ``heads_per_group`` heads sharing a group's q and k; v [N, heads * dv].  With ``m_tok`` [N, heads] the
    state has one more value column, the normalizer n <- a_t n + b_t k_t, and
    o_t <- o_t / (max(|n . q_t|, exp(-m_tok)) + 1e-6).  Everything is computed in float32; the order of every
    sum depends on dk alone, so any cut of a prompt gives the same numbers.  ``max_len``: the most tokens that a
    sequence brings; with ``ws`` (a Workspace, for scratch) steps of ``SCAN_CHUNKED_FROM`` tokens a sequence and
    more take the kernels that walk a sequence in chunks of 32 tokens, whose sums come in another order (the
    results differ from the token-by-token kernel's by rounding)."""
    N = out.shape[0]
    if not 1 <= dk <= MAX_SCAN_KEY_DIM:
        raise KernelError(f"scalar_scan: key size {dk} is outside 1..{MAX_SCAN_KEY_DIM}")
    if heads_per_group < 1 or n_heads % heads_per_group:
        raise KernelError(f"scalar_scan: {n_heads} heads do not split into groups of {heads_per_group}")
    groups = n_heads // heads_per_group
    qp, ldq = _cols(q, "scalar_scan q", N, groups * dk)
    kp, ldk = _cols(k, "scalar_scan k", N, groups * dk)
    vp, ldv = _cols(v, "scalar_scan v", N, n_heads * dv)
    ap, lda = _cols(log_a, "scalar_scan log decay", N, n_heads)
    bp, ldb = _cols(b, "scalar_scan input factor", N, n_heads)
    norm = m_tok is not None
    _need(state, "scalar_scan state", torch.float32, (None, n_heads, dv + (1 if norm else 0), dk))
    _guard("core", "scalar_scan", out.device, n_slots=state.shape[0])
    if ws is not None and max_len >= SCAN_CHUNKED_FROM:
        chunks = int(_fn("core", "mv_scalar_chunks")(N, int(n_seqs)))
        G = ws.get("scalar_scan_products", (chunks, groups, SCAN_CHUNK, SCAN_CHUNK), torch.float32)
        o_aug = ws.get("scalar_scan_o_aug", (N, n_heads * (dv + 1)), torch.float32) if norm else None
        _check(_fn("core", "mv_scalar_scan_chunked")(
            qp, ldq, kp, ldk, vp, ldv, ap, lda, bp, ldb, _need(skip, "scalar_scan skip", torch.float32, (n_heads,), True),
            _need(m_tok, "scalar_scan m", torch.float32, (N, n_heads), True), float(q_scale), state.data_ptr(),
            _need(slots, "slots", torch.int32), _need(cu, "cu", torch.int32),
            _need(out, "scalar_scan out", torch.float32, (N, n_heads * dv)), G.data_ptr(),
            o_aug.data_ptr() if norm else None, N, int(n_seqs), int(max_len), n_heads, int(heads_per_group), dk, dv,
            int(norm), _stream()), "mv_scalar_scan_chunked")
        add_launches(1 if norm else 0)
        account(N * n_heads * (2 * dk // heads_per_group + 2 * dv) * 4 + 2 * n_seqs * n_heads * dk * dv * 4
                + 2 * chunks * groups * SCAN_CHUNK * SCAN_CHUNK * 4,
                4 * N * n_heads * dk * dv + N * n_heads * SCAN_CHUNK * dv + N * groups * SCAN_CHUNK * dk)
        return out
    _check(_fn("core", "mv_scalar_scan")(
        qp, ldq, kp, ldk, vp, ldv, ap, lda, bp, ldb, _need(skip, "scalar_scan skip", torch.float32, (n_heads,), True),
        _need(m_tok, "scalar_scan m", torch.float32, (N, n_heads), True), float(q_scale), state.data_ptr(),
        _need(slots, "slots", torch.int32), _need(cu, "cu", torch.int32),
        _need(out, "scalar_scan out", torch.float32, (N, n_heads * dv)), int(n_seqs), n_heads, int(heads_per_group), dk, dv,
        int(norm), _stream()), "mv_scalar_scan")
    account(N * n_heads * (2 * dk + 2 * dv) * 4 + 2 * n_seqs * n_heads * dk * dv * 4, 4 * N * n_heads * dk * dv)
    return out


def memory_gates(zi: torch.Tensor, zf: torch.Tensor, bi: torch.Tensor, bf: torch.Tensor, cap: float,
                 m_state: torch.Tensor, slots: torch.Tensor, cu: torch.Tensor, log_a: torch.Tensor, b: torch.Tensor,
                 m_tok: torch.Tensor, n_seqs: int, n_heads: int) -> None:
    """The log gates of a matrix memory: i = cap tanh((zi + bi) / cap), f = log sigmoid(cap tanh((zf + bf) / cap)),
    the running maximum m_t = max(f_t + m_(t-1), i_t) from and into ``m_state`` [slots, heads], and from them
    log_a = f + m_(t-1) - m_t, b = exp(i - m_t), m_tok = m_t, all float32 [N, heads]."""
    N = log_a.shape[0]
    ip, ldi = _cols(zi, "memory_gates input gate", N, n_heads)
    fp, ldf = _cols(zf, "memory_gates forget gate", N, n_heads)
    _guard("core", "scalar_scan", log_a.device, n_slots=m_state.shape[0])
    _check(_fn("core", "mv_memory_gates")(
        ip, ldi, fp, ldf, _need(bi, "input gate bias", torch.float32, (n_heads,)),
        _need(bf, "forget gate bias", torch.float32, (n_heads,)), float(cap),
        _need(m_state, "memory_gates m", torch.float32, (None, n_heads)), _need(slots, "slots", torch.int32),
        _need(cu, "cu", torch.int32), _need(log_a, "log_a", torch.float32, (N, n_heads)),
        _need(b, "b", torch.float32, (N, n_heads)), _need(m_tok, "m_tok", torch.float32, (N, n_heads)), int(n_seqs),
        n_heads, _stream()), "mv_memory_gates")
    account(N * n_heads * 20)


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                seq_of: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, n_seqs: int,
                act: bool = False, one_each: bool = False) -> torch.Tensor:
    """out = bias + sum_j taps[:, j] * u[t - (K - 1) + j] per channel along each sequence (the last tap is the
    current token's; zeros before a sequence's start), float32; with ``act`` silu of that.  ``u`` [N, C] may be a
    column slice; ``state`` [slots, K - 1, C] holds each sequence's last K - 1 inputs and is brought up to date.
    ``one_each``: every sequence brings one token and row b is sequence b's (a decode step): output and kept inputs in
    one kernel."""
    N, C = out.shape
    K = taps.shape[1]
    if not 1 <= K <= MAX_CONV_K:
        raise KernelError(f"causal_conv: {K} taps are outside 1..{MAX_CONV_K}")
    one_each = bool(one_each) and N == int(n_seqs)
    up, ldu = _cols(u, "causal_conv input", N, C)
    if K > 1:
        _guard("core", "state_space", out.device, n_slots=state.shape[0])
    _check(_fn("core", "mv_causal_conv")(
        up, ldu, _need(taps, "conv taps", torch.float32, (C, K)), _need(bias, "conv bias", torch.float32, (C,), True),
        _need(state, "conv state", torch.float32, (None, max(K - 1, 0), C)) if K > 1 else None,
        _need(seq_of, "seq_of", torch.int32), _need(cu, "cu", torch.int32), _need(slots, "slots", torch.int32),
        _need(out, "causal_conv out", torch.float32), N, int(n_seqs), C, K, int(bool(act)), int(one_each), _stream()),
        "mv_causal_conv")
    if one_each or K == 1:
        add_launches(-1)                     # one kernel, not the two that a call is counted as
    account(N * C * 8 + 2 * n_seqs * (K - 1) * C * 4, 2 * N * C * K)
    return out


def causal_conv_silu(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                     seq_of: torch.Tensor, cu: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, n_seqs: int,
                     one_each: bool = False) -> torch.Tensor:
    """:func:`causal_conv` followed by silu."""
    return causal_conv(u, taps, bias, state, seq_of, cu, slots, out, n_seqs, act=True, one_each=one_each)


def step_size(raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, log_a: torch.Tensor, b: torch.Tensor) -> None:
    """dt = softplus(raw + dt_bias) per token and head; b = dt, log_a = -exp(a_log) * dt; float32 [N, heads]."""
    N, H = log_a.shape
    rp, ldr = _cols(raw, "step_size raw", N, H)
    _check(_fn("core", "mv_step_size")(
        rp, ldr, _need(dt_bias, "dt bias", torch.float32, (H,)), _need(a_log, "A_log", torch.float32, (H,)),
        _need(log_a, "log_a", torch.float32), _need(b, "b", torch.float32, (N, H)), N, H, _stream()), "mv_step_size")
    account(N * H * 12)


def ssm_decode_prepare(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
                       slots: torch.Tensor, out: torch.Tensor, raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
                       log_a: torch.Tensor, b: torch.Tensor) -> None:
    """:func:`causal_conv_silu` and :func:`step_size` in one kernel for a step of one token a sequence (row i of
    the step is the token of ``slots[i]``)."""
    N, C = out.shape
    K, H = taps.shape[1], log_a.shape[1]
    if not 1 <= K <= MAX_CONV_K:
        raise KernelError(f"ssm_decode_prepare: {K} taps are outside 1..{MAX_CONV_K}")
    if slots.numel() != N:
        raise KernelError(f"ssm_decode_prepare: {N} rows for {slots.numel()} sequences; this kernel takes one token a sequence")
    up, ldu = _cols(u, "ssm_decode_prepare input", N, C)
    rp, ldr = _cols(raw, "ssm_decode_prepare step sizes", N, H)
    _guard("core", "state_space", out.device, n_slots=state.shape[0])
    _check(_fn("core", "mv_ssm_decode_prepare")(
        up, ldu, _need(taps, "conv taps", torch.float32, (C, K)), _need(bias, "conv bias", torch.float32, (C,), True),
        _need(state, "conv state", torch.float32, (None, K - 1, C)) if K > 1 else None, _need(slots, "slots", torch.int32),
        _need(out, "conv out", torch.float32), N, C, K, rp, ldr, _need(dt_bias, "dt bias", torch.float32, (H,)),
        _need(a_log, "A_log", torch.float32, (H,)), _need(log_a, "log_a", torch.float32, (N, H)),
        _need(b, "b", torch.float32, (N, H)), H, _stream()), "mv_ssm_decode_prepare")
    account(N * (C * 8 + H * 12) + 2 * N * (K - 1) * C * 4, 2 * N * C * K)


MAX_EXPERTS = 1024


ROUTE_SIGMOID, ROUTE_SOFTMAX = 0, 1


def route(z: torch.Tensor, dense: torch.Tensor, pick: torch.Tensor, pick_w: torch.Tensor, n_experts: int,
          n_groups: int, keep: int, top: int, shared_gate: bool, *, mode: int = ROUTE_SIGMOID,
          correction: Optional[torch.Tensor] = None, out_scale: float = 1.0, n_identity: int = 0) -> None:
    """Router of a mixture of experts from float32 logits ``z`` [N, routed (+ 1)]: scores sigmoid(z), or with
    ``ROUTE_SOFTMAX`` softmax(z) over all routed entries; the entries
    form ``n_groups`` equal groups of neighbours whose score is the sum of their two largest scores; among the
    entries of the ``keep`` best groups the ``top`` largest are chosen, with weights score / (sum of the chosen
    scores + 1e-20) * ``out_scale``.  ``correction`` [routed] is added to the scores for the choice only.
    ``n_experts`` counts all routed entries; its last ``n_identity`` are identity experts.  ``dense``
    [N, routed (+ 1)] gets a row of weights (zero where not chosen), laid out [experts | with ``shared_gate``
    sigmoid of the last logit | identity experts]; ``pick`` / ``pick_w`` [N, top] the lists (routed indices)."""
    N = dense.shape[0]
    E = int(n_experts)
    cols = E + (1 if shared_gate else 0)
    if (E < 1 or E > MAX_EXPERTS or n_groups < 1 or E % n_groups or not 1 <= keep <= n_groups or not 1 <= top <= 32
            or top > keep * (E // n_groups) or not 0 <= n_identity <= E):
        raise KernelError(f"route: {E} experts in {n_groups} groups, {keep} groups kept, {top} chosen: not a routing "
                          f"this kernel takes (at most {MAX_EXPERTS} experts, 32 chosen)")
    zp, ldz = _cols(z, "router logits", N, cols)
    _check(_fn("core", "mv_route")(
        zp, ldz, _need(dense, "route weights", torch.float32, (N, cols)), _need(pick, "route picks", torch.int32, (N, top)),
        _need(pick_w, "route pick weights", torch.float32, (N, top)), N, E, int(n_groups), int(keep), int(top),
        int(bool(shared_gate)), int(mode), _need(correction, "route correction", torch.float32, (E,), True),
        float(out_scale), int(n_identity), _stream()), "mv_route")
    account(N * cols * 8)


def identity_experts(h: torch.Tensor, dense: torch.Tensor, col0: int, n_cols: int, resid: torch.Tensor,
                     accumulate: bool = True) -> torch.Tensor:
    """resid[n] (+)= (dense[n, col0] + ... + dense[n, col0 + n_cols - 1]) * h[n]: the experts whose output is
    their input, with the router's weights from its dense rows."""
    N, H = h.shape
    if dense.dim() != 2 or dense.shape[0] != N or col0 < 0 or col0 + n_cols > dense.shape[1]:
        raise KernelError(f"identity_experts: columns {col0}..{col0 + n_cols} of weights {tuple(dense.shape)} for {N} rows")
    _check(_fn("core", "mv_identity_experts")(
        _need(h, "identity_experts input"), _dt(h), _need(dense, "route weights", torch.float32), dense.shape[1], int(col0),
        int(n_cols), _need(resid, "residual stream", torch.float32, (N, H)), N, H, int(bool(accumulate)), _stream()),
        "mv_identity_experts")
    account(N * H * (8 + h.element_size()))
    return resid


def routed_glu(gu: torch.Tensor, dense: torch.Tensor, hid: torch.Tensor, n_experts: int, ff: int, shared_ff: int,
               group: int = 0, shared_group: int = 0, extra_cols: int = 0) -> torch.Tensor:
    """hid[n, c] = weight(n, expert of column c) * silu(gate[n, c]) * up[n, c] over the columns of all experts end to
    end (then a shared expert's), from ``gu`` [N, 2 * F] float32 and the router's dense weights; nothing is computed
    where the weight is zero.  ``gu`` holds each expert's gates and ups together, [e * 2 ff, (e + 1) * 2 ff): the gates,
    then the ups, or with ``group`` 16 alternating in groups of 16 columns; the shared expert's block likewise with
    ``shared_group``."""
    N, F = hid.shape
    if F != n_experts * ff + shared_ff:
        raise KernelError(f"routed_glu: {F} columns for {n_experts} experts of {ff} and a shared one of {shared_ff}")
    if (group and ff % group) or (shared_group and shared_ff % shared_group):
        raise KernelError(f"routed_glu: widths {ff} and {shared_ff} against groups of {group} and {shared_group}")
    _check(_fn("core", "mv_routed_glu")(
        _need(gu, "routed_glu input", torch.float32, (N, 2 * F)),
        _need(dense, "route weights", torch.float32, (N, n_experts + (1 if shared_ff else 0) + extra_cols)),
        _need(hid, "routed_glu out"), _dt(hid), N, int(n_experts), int(ff), int(shared_ff), int(group), int(shared_group),
        int(extra_cols), _stream()), "mv_routed_glu")
    account(N * F * (8 + hid.element_size()))
    return hid


def scale_expert_columns(h: torch.Tensor, dense: torch.Tensor, n_experts: int, ff: int, shared_ff: int,
                         extra_cols: int = 0) -> torch.Tensor:
    """h[n, c] *= weight(n, expert of column c) in place, over the columns of all experts end to end (then a shared
    expert's): for activations that a product's epilogue has gated already."""
    N, F = h.shape
    if F != n_experts * ff + shared_ff:
        raise KernelError(f"scale_expert_columns: {F} columns for {n_experts} experts of {ff} and a shared one of {shared_ff}")
    _check(_fn("core", "mv_scale_expert_columns")(
        _need(h, "gated activations"), _dt(h),
        _need(dense, "route weights", torch.float32, (N, n_experts + (1 if shared_ff else 0) + extra_cols)),
        N, int(n_experts), int(ff), int(shared_ff), int(extra_cols), _stream()), "mv_scale_expert_columns")
    account(2 * N * F * h.element_size())
    return h


GROUPED_TILE_ROWS = 128


def grouped_tiles(n_entries: int, n_experts: int) -> int:
    """Tiles of ``GROUPED_TILE_ROWS`` rows that the sorted entries can need at most, every expert's run padded to
    whole tiles."""
    return (n_entries + n_experts * (GROUPED_TILE_ROWS - 1)) // GROUPED_TILE_ROWS + 1


def expert_sort(pick: torch.Tensor, n_experts: int, x: torch.Tensor, rank: torch.Tensor, counts: torch.Tensor,
                place: torch.Tensor, xs: torch.Tensor, offsets: Optional[torch.Tensor] = None,
                tile_group: Optional[torch.Tensor] = None) -> None:
    """The (token, choice) entries of ``pick`` [N, top] sorted by expert (stable): ``counts`` [experts] entries an
    expert, ``place`` [N * top] where each entry went, and the tokens' rows of ``x`` [N, H] copied to ``xs`` in that
    order, so that an expert's rows lie together.  With ``offsets`` [experts] and ``tile_group`` [tiles] every
    expert's run starts on a tile of ``GROUPED_TILE_ROWS`` rows (``xs`` then has tiles * that many rows, the rows
    between runs are left as they are), ``offsets`` says where, and ``tile_group`` names each tile's expert (-1 for
    the spare tiles at the end): what :func:`gemm_tc_grouped` takes."""
    N, top = pick.shape
    H = x.shape[1]
    padded = offsets is not None
    if padded != (tile_group is not None):
        raise KernelError("expert_sort: offsets and tile_group come together")
    rows = tile_group.numel() * GROUPED_TILE_ROWS if padded else N * top
    if padded and tile_group.numel() < grouped_tiles(N * top, n_experts):
        raise KernelError(f"expert_sort: {tile_group.numel()} tiles for {N * top} entries of {n_experts} experts")
    _check(_fn("core", "mv_expert_rank")(
        _need(pick, "picks", torch.int32), N * top, int(n_experts), _need(rank, "ranks", torch.int32, (N * top,)),
        _need(counts, "counts", torch.int32, (n_experts,)), _stream()), "mv_expert_rank")
    if padded:
        _check(_fn("core", "mv_expert_tiles")(
            counts.data_ptr(), int(n_experts), GROUPED_TILE_ROWS, _need(offsets, "offsets", torch.int32, (n_experts,)),
            _need(tile_group, "tile groups", torch.int32), tile_group.numel(), _stream()), "mv_expert_tiles")
    _check(_fn("core", "mv_expert_gather")(
        pick.data_ptr(), rank.data_ptr(), counts.data_ptr(), offsets.data_ptr() if padded else None,
        _need(x, "expert_sort rows", None, (N, H)), _dt(x), N, top, H,
        _need(place, "places", torch.int32, (N * top,)), _need(xs, "sorted rows", x.dtype, (rows, H)), _stream()),
        "mv_expert_gather")
    account(N * (1 + top) * H * x.element_size())


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, n: int, k: int, *,
                    row_step: int = 0, k_step: int = 0, swiglu: bool = False, active_rows: Optional[int] = None) -> torch.Tensor:
    """One product for many groups, on the tcgen05 tensor cores (bfloat16): the rows of ``x`` [tiles * 128, k] are
    sorted by group with every group's run padded to whole tiles (:func:`expert_sort`), ``tile_group`` names each
    tile's group (negative: nothing to do), and ``w`` holds the groups' [n, k] matrices one below the other
    (``row_step`` rows a group) or side by side along its columns (``k_step`` columns a group).  ``out``
    [tiles * 128, n] float32 or bfloat16, or with ``swiglu`` bfloat16 [tiles * 128, n / 2] from rows of ``w`` that
    alternate in groups of 16 gate and 16 up rows.  ``active_rows``: rows that belong to a group, for the profile's
    accounts."""
    M = x.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_grouped: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if M != tile_group.numel() * GROUPED_TILE_ROWS or x.shape[1] != k:
        raise KernelError(f"gemm_tc_grouped: x is {tuple(x.shape)} for {tile_group.numel()} tiles and k = {k}")
    if k % 8 or k_step % 8 or (row_step and k_step):
        raise KernelError(f"gemm_tc_grouped: k {k} and k_step {k_step} must be multiples of 8; one of row_step and k_step")
    if swiglu:
        if n % 32:
            raise KernelError(f"gemm_tc_grouped: the SwiGLU epilogue needs rows in groups of 32, got {n}")
        mode, ldo = 3, n // 2
        _need(out, "gemm out", torch.bfloat16, (M, n // 2))
    else:
        mode, ldo = (0 if out.dtype == torch.float32 else 1), n
        _need(out, "gemm out", None, (M, n))
        _dt(out)
    _check(_fn("bf16", "mv_gemm_tc_grouped")(
        _need(x, "gemm x"), _need(w, "gemm w"), out.data_ptr(), mode, M, int(n), int(k), ldo, w.shape[0], w.shape[1],
        _need(tile_group, "tile groups", torch.int32), int(row_step), int(k_step), _error_flag(x.device).data_ptr(),
        _stream()), "mv_gemm_tc_grouped")
    rows = M if active_rows is None else active_rows
    account(rows * (k * 2 + ldo * out.element_size()) + _nbytes(w), 2 * rows * n * k)
    return out


def expert_combine(ys: torch.Tensor, place: torch.Tensor, pick_w: torch.Tensor, shared: Optional[torch.Tensor],
                   gate: Optional[torch.Tensor], out: torch.Tensor, accumulate: bool) -> torch.Tensor:
    """out[n] (+)= sum_k pick_w[n, k] * ys[place[n * top + k]] (+ gate[n] * shared[n]), float32: the chosen experts'
    results gathered back in the order of the choices.  ``gate`` [N, 1] may be a column of a wider matrix.  ``ys``
    has at least N * top rows (more where the experts' runs are padded)."""
    N, H = out.shape
    top = pick_w.shape[1]
    if ys.shape[0] < N * top:
        raise KernelError(f"expert_combine: {ys.shape[0]} result rows for {N * top} entries")
    gp, ldg = _cols(gate, "shared gate", N, 1) if gate is not None else (None, 0)
    _check(_fn("core", "mv_expert_combine")(
        _need(ys, "expert results", torch.float32, (None, H)), _need(place, "places", torch.int32, (N * top,)),
        _need(pick_w, "pick weights", torch.float32, (N, top)), _need(shared, "shared result", torch.float32, (N, H), True),
        gp, ldg, _need(out, "combine out", torch.float32), N, top, H, int(bool(accumulate)), _stream()), "mv_expert_combine")
    account(N * H * 4 * (top + 2 + (1 if shared is not None else 0)))
    return out


MAX_SCAN_KEY_DIM = 256
SCAN_ACT_NONE, SCAN_ACT_SILU = 0, 1
SCAN_CHUNKED_FROM = 16          # a step whose longest sequence brings this many tokens walks them in chunks
SCAN_CHUNK = 32


def _cols(t: torch.Tensor, name: str, n_rows: int, width: int):
    """Pointer and row stride of a float32 matrix that may be a column slice of a wider one."""
    if (not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.shape[0] != n_rows or t.shape[1] != width
            or (t.stride(1) != 1 and width > 1)):
        raise KernelError(f"{name}: needs float32 [{n_rows}, {width}] on a CUDA device with unit column stride, got "
                          f"{t.dtype} {tuple(t.shape)} strides {t.stride()} on {t.device}")
    return t.data_ptr(), t.stride(0)


def decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, slots: torch.Tensor,
               cu: torch.Tensor, out: torch.Tensor, n_seqs: int, n_heads: int, dk: int, dv: int, *,
               decay_logits: Optional[torch.Tensor] = None, inv_tau: float = 1.0,
               head_decay: Optional[torch.Tensor] = None, q_scale: float = 1.0, act: int = SCAN_ACT_NONE,
               max_len: int = 1, ws=None) -> torch.Tensor:
    """Linear attention with a decaying state, per head: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t, over the
    step's tokens in order, from and into ``state`` [slots, heads, dv, dk] (float32, transposed: a value
    column's key channels lie together).  The decay a_t is sigmoid(decay_logits)^inv_tau per token and key
    channel, or ``head_decay`` [heads], a constant per head.  q, k [N, heads * dk] and v [N, heads * dv] are
    float32 and may be column slices of one wider matrix; ``act`` is applied to all three as they are read
    and ``q_scale`` multiplies q.  Everything is computed in float32.  ``max_len``: the most tokens that a
    sequence brings; with ``ws`` (a Workspace, for scratch) steps of ``SCAN_CHUNKED_FROM`` tokens a sequence and
    more take the kernels that walk a sequence in chunks of 32 tokens, whose sums come in another order (the
    results differ from the token-by-token kernel's by rounding)."""
    N = out.shape[0]
    if not 1 <= dk <= MAX_SCAN_KEY_DIM:
        raise KernelError(f"decay_scan: key size {dk} is outside 1..{MAX_SCAN_KEY_DIM}")
    if (decay_logits is None) == (head_decay is None):
        raise KernelError("decay_scan: give either decay logits per token and channel or a decay per head")
    qp, ldq = _cols(q, "decay_scan q", N, n_heads * dk)
    kp, ldk = _cols(k, "decay_scan k", N, n_heads * dk)
    vp, ldv = _cols(v, "decay_scan v", N, n_heads * dv)
    zp, ldz = _cols(decay_logits, "decay_scan decay logits", N, n_heads * dk) if decay_logits is not None else (None, 0)
    _need(state, "decay_scan state", torch.float32, (None, n_heads, dv, dk))
    _guard("core", "decay_scan", out.device, n_slots=state.shape[0])
    if ws is not None and max_len >= SCAN_CHUNKED_FROM:
        chunks = int(_fn("core", "mv_decay_chunks")(N, int(n_seqs)))
        qd = ws.get("scan_qd", (N, n_heads * dk), torch.float32)
        kd = ws.get("scan_kd", (N, n_heads * dk), torch.float32)
        ed = ws.get("scan_ed", (chunks, n_heads * dk), torch.float32)
        pm = ws.get("scan_p", (chunks, n_heads, SCAN_CHUNK, SCAN_CHUNK), torch.float32)
        _check(_fn("core", "mv_decay_scan_chunked")(
            qp, ldq, kp, ldk, vp, ldv, zp, ldz, _need(head_decay, "head decay", torch.float32, (n_heads,), True),
            float(inv_tau), float(q_scale), int(act), state.data_ptr(), _need(slots, "slots", torch.int32),
            _need(cu, "cu", torch.int32), _need(out, "decay_scan out", torch.float32, (N, n_heads * dv)),
            qd.data_ptr(), kd.data_ptr(), ed.data_ptr(), pm.data_ptr(), int(n_seqs), int(max_len), n_heads, dk, dv,
            _stream()), "mv_decay_scan_chunked")
        account(N * n_heads * (6 * dk + 2 * dv) * 4 + 2 * n_seqs * n_heads * dk * dv * 4, 5 * N * n_heads * dk * dv)
        return out
    _check(_fn("core", "mv_decay_scan")(
        qp, ldq, kp, ldk, vp, ldv, zp, ldz, _need(head_decay, "head decay", torch.float32, (n_heads,), True),
        float(inv_tau), float(q_scale), int(act), state.data_ptr(), _need(slots, "slots", torch.int32),
        _need(cu, "cu", torch.int32), _need(out, "decay_scan out", torch.float32, (N, n_heads * dv)), int(n_seqs),
        n_heads, dk, dv, _stream()), "mv_decay_scan")
    account(N * n_heads * (2 * dk + 2 * dv) * 4 + 2 * n_seqs * n_heads * dk * dv * 4, 4 * N * n_heads * dk * dv)
    return out


def kv_page_elems(nkv: int, page_size: int, dk: int, dv: int) -> int:
    """Elements of one layer's page when keys and values differ in size: [kv head][row][dk] keys, then
    [kv head][row][dv] values."""
    return nkv * page_size * (dk + dv)


def _check_kv_wide(pool: torch.Tensor, nkv: int, page_size: int, dk: int, dv: int, what: str) -> None:
    if dk == dv and pool.dim() == 5:
        _check_kv(pool, nkv, dk, page_size, what)
        return
    if pool.dim() != 2 or pool.shape[1] != kv_page_elems(nkv, page_size, dk, dv):
        raise KernelError(f"{what}: cache pool shape {tuple(pool.shape)}, expected [pages, "
                          f"{kv_page_elems(nkv, page_size, dk, dv)}] ({nkv} kv heads x {page_size} rows x ({dk} + {dv}))")
    if page_size & (page_size - 1):
        raise KernelError(f"{what}: page size {page_size} is not a power of two")


def qkv_prepare_wide(proj: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                     rot_dims: int, inv_freq: Optional[torch.Tensor], positions, seq_of, page_table,
                     pool: torch.Tensor, page_size: int, q_out: torch.Tensor, nh: int, nkv: int, dk: int,
                     dv: int, *, per_head: bool = False, amplitude: float = 1.0) -> torch.Tensor:
    """From a row [q | k | v | ...] of a fused projection (float32, any row stride): root-mean-square norm over
    the whole of q and the whole of k (weights wq [nh * dk], wk [nkv * dk]; None: no norm), or with
    ``per_head`` over every head by itself (weights wq, wk [dk], shared by the heads); rotation of the
    first ``rot_dims`` elements of every head (element i with i + rot_dims / 2, angle pos * inv_freq[i], cos and
    sin times ``amplitude``), q out in the model's dtype, k and v into the token's row of its page."""
    N = q_out.shape[0]
    need = nh * dk + nkv * (dk + dv)
    if (not proj.is_cuda or proj.dtype != torch.float32 or proj.dim() != 2 or proj.shape[0] != N or proj.shape[1] < need
            or proj.stride(1) != 1):
        raise KernelError(f"qkv_prepare_wide: projection must be float32 [{N}, >= {need}], got {proj.dtype} "
                          f"{tuple(proj.shape)}")
    if rot_dims % 2 or not 0 <= rot_dims <= dk:
        raise KernelError(f"qkv_prepare_wide: {rot_dims} rotated elements in heads of {dk}")
    _check_kv_wide(pool, nkv, page_size, dk, dv, "qkv_prepare_wide")
    if pool.dtype != q_out.dtype:
        raise KernelError(f"qkv_prepare_wide: cache is {pool.dtype} but q is {q_out.dtype}")
    _guard("core", "attention_sink", proj.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_qkv_prepare_wide")(
        proj.data_ptr(), proj.stride(0), _need(wq, "q norm weight", torch.float32, (dk if per_head else nh * dk,), True),
        _need(wk, "k norm weight", torch.float32, (dk if per_head else nkv * dk,), True), float(eps), int(rot_dims),
        _need(inv_freq, "inv_freq", torch.float32, (rot_dims // 2,), rot_dims == 0),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size, _need(pool, "cache pool"),
        pool.stride(0), _need(q_out, "q out", None, (N, nh * dk)), _dt(q_out), N, nh, nkv, dk, dv, int(bool(per_head)),
        float(amplitude), _stream()), "mv_qkv_prepare_wide")
    account(N * need * 4 + N * (nh * dk + nkv * (dk + dv)) * q_out.element_size())
    return q_out


def attention_sink(q: torch.Tensor, pool: torch.Tensor, page_size: int, page_table, positions, seq_of,
                   out: torch.Tensor, nh: int, nkv: int, dk: int, dv: int, scale: float, *, softcap: float = 0.0,
                   window: int = 0, keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None, head_tile: int = 0, chunk: int = 0,
                   distance_bias: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, values_in_keys: bool = False,
                   gate_wide: bool = False, out_all: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal softmax attention of every token of the step over its sequence's cache (which already holds the
    step's own keys), keys of size dk and values of size dv.  ``softcap`` c > 0: s <- c tanh(s / c).  ``window``
    w > 0 with ``keep_first`` f: query i reads key j if i - j < w or j < f.  ``sinks`` [nh]: exp(sink) joins
    each head's denominator.  ``gate``: float32 logits [N, nh] (a column slice is fine); the head's output is
    multiplied by sigmoid(gate).  ``chunk`` c > 0 (instead of a window): query i reads key j <= i only if
    i // c == j // c.  ``head_tile``: how many query heads of a kv head share a block and its loads
    (1, 2 or 4; 0: the kernel chooses by the step's size).  ``distance_bias`` (r1, r2), float32 [nh] each:
    r1_h ln(1 + r2_h (i - j)) is taken off the score.  ``values_in_keys``: the values are the first dv elements of
    the key rows and a page holds key rows only.  ``gate_wide``: ``gate`` is [N, nh * dv], one logit an element.
    ``out_all``: float32 [N, nh, nkv, dv]; every head's weights are applied to the values of every kv head and
    written there (``out`` is then left alone): what :func:`mix_heads` needs."""
    N = q.shape[0]
    if not (1 <= dk <= MAX_HEAD_DIM and 1 <= dv <= MAX_HEAD_DIM):
        raise KernelError(f"attention_sink: key size {dk} and value size {dv} must lie in 1..{MAX_HEAD_DIM}")
    if nkv < 1 or nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    _check_kv_wide(pool, nkv, page_size, dk, 0 if values_in_keys else dv, "attention_sink")
    if q.dtype != pool.dtype or (out_all is None and out.dtype != q.dtype):
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    gp, ldg = _cols(gate, "attention gate", N, nh * dv if gate_wide else nh) if gate is not None else (None, 0)
    r1, r2 = _bias_pair(distance_bias, nh, values_in_keys, dk, dv)
    _guard("core", "attention_sink", q.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_attention_sink")(
        _need(q, "q", None, (N, nh * dk)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(sinks, "sinks", torch.float32, (nh,), True), gp, ldg,
        _need(out, "attention out", None, (N, nh * dv), out_all is not None),
        _dt(q), N, nh, nkv, dk, dv, float(scale), float(softcap), int(window), int(keep_first), int(head_tile),
        int(chunk), r1, r2, int(bool(values_in_keys)), int(bool(gate_wide)),
        _need(out_all, "attention out of all kv heads", torch.float32, (N, nh, nkv, dv), True), _stream()), "mv_attention_sink")
    return out if out_all is None else out_all


def _bias_pair(distance_bias, nh: int, values_in_keys: bool, dk: int, dv: int):
    if values_in_keys and dv > dk:
        raise KernelError(f"attention: values of {dv} cannot be the first elements of keys of {dk}")
    if distance_bias is None:
        return None, None
    r1, r2 = distance_bias
    return _need(r1, "distance bias r1", torch.float32, (nh,)), _need(r2, "distance bias r2", torch.float32, (nh,))


def mix_heads(o_all: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, nh: int, nkv: int, dv: int) -> torch.Tensor:
    """out[n, h, :] = sum_g talk[h, g] * o_all[n, g, kv head of h, :]: attention whose softmax weights are mixed
    between the heads after the softmax, w'_h = sum_g talk[h, g] w_g, each head applying its mixed weights to the
    values of its own kv head; ``o_all`` float32 [N, nh, nkv, dv] holds every head's weights applied to every kv
    head's values (:func:`attention_sink` with ``out_all``); ``talk`` float32 [nh, nh]; ``out`` [N, nh * dv]."""
    N = out.shape[0]
    if nkv < 1 or nh % nkv:
        raise KernelError(f"mix_heads: {nh} heads are not a multiple of {nkv} kv heads")
    _check(_fn("core", "mv_mix_heads")(
        _need(o_all, "mix_heads input", torch.float32, (N, nh, nkv, dv)), _need(talk, "mix_heads talk", torch.float32, (nh, nh)),
        _need(out, "mix_heads out", None, (N, nh * dv)), _dt(out), N, nh, nkv, dv, _stream()), "mv_mix_heads")
    account(N * nh * dv * (4 * nkv + out.element_size()), 2 * N * nh * nh * dv)
    return out


def attention_sink_prefill_supported(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """What the tensor-core kernel for steps of many query tokens takes: bfloat16, key and value sizes that are
    multiples of 16 up to 128."""
    return (dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and 16 <= dk <= PREFILL_ATTENTION_MAX_HEAD_DIM
            and 16 <= dv <= PREFILL_ATTENTION_MAX_HEAD_DIM)


def attention_sink_prefill(q: torch.Tensor, pool: torch.Tensor, page_size: int, page_table, cu, starts,
                           out: torch.Tensor, n_seqs: int, nh: int, nkv: int, dk: int, dv: int, scale: float, *,
                           softcap: float = 0.0, window: int = 0, keep_first: int = 0,
                           sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                           chunk: int = 0, distance_bias: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                           values_in_keys: bool = False, gate_wide: bool = False,
                           out_all: Optional[torch.Tensor] = None, split_weights: bool = False) -> torch.Tensor:
    """:func:`attention_sink` for a step with many query tokens, on the tensor cores (bfloat16, key and value
    sizes 16..128 in steps of 16).  The step's tokens are packed sequence by sequence (``cu``), sequence b
    starting at position ``starts[b]``.  ``split_weights``: a softmax weight enters the value product as two
    bfloat16 numbers (the rounded weight and what the rounding left), 16 bits of its mantissa instead of 8."""
    N = q.shape[0]
    if not attention_sink_prefill_supported(q.dtype, dk, dv):
        raise KernelError(f"attention_sink_prefill: needs bfloat16 and key and value sizes 16..128 in steps of 16, "
                          f"got {q.dtype}, {dk}, {dv}")
    if nkv < 1 or nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    _check_kv_wide(pool, nkv, page_size, dk, 0 if values_in_keys else dv, "attention_sink_prefill")
    if q.dtype != pool.dtype or (out_all is None and out.dtype != q.dtype):
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    gp, ldg = _cols(gate, "attention gate", N, nh * dv if gate_wide else nh) if gate is not None else (None, 0)
    r1, r2 = _bias_pair(distance_bias, nh, values_in_keys, dk, dv)
    _guard("bf16", "attention_sink_prefill", q.device, n_pages=pool.shape[0])
    _check(_fn("bf16", "mv_attention_sink_prefill")(
        _need(q, "q", None, (N, nh * dk)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32),
        _need(sinks, "sinks", torch.float32, (nh,), True), gp, ldg,
        _need(out, "attention out", None, (N, nh * dv), out_all is not None),
        N, n_seqs, nh, nkv, dk, dv, float(scale), float(softcap), int(window), int(keep_first), int(chunk), r1, r2,
        int(bool(values_in_keys)), int(bool(gate_wide)),
        _need(out_all, "attention out of all kv heads", torch.float32, (N, nh, nkv, dv), True), int(bool(split_weights)),
        _stream()), "mv_attention_sink_prefill")
    return out if out_all is None else out_all


def embed_bigram(table: torch.Tensor, bigram: torch.Tensor, tokens, positions, seq_of, cu, slots, prev: torch.Tensor,
                 out: torch.Tensor, kept: Optional[torch.Tensor], mul_prev: int, mul_cur: int) -> torch.Tensor:
    """out[n] = table[token] + bigram[r] in float32, r = (previous token * mul_prev + token * mul_cur) mod buckets with
    buckets = rows of ``bigram`` - 1, or the last row for a token at position 0.  ``prev`` int32 [slots]: the last
    token of each sequence before this step; it is brought up to date.  ``kept``: a second copy of the rows, or None."""
    N = tokens.numel()
    V, H = table.shape
    if bigram.dim() != 2 or bigram.shape[1] != H or bigram.shape[0] < 2 or bigram.dtype != table.dtype:
        raise KernelError(f"embed_bigram: bigram table {tuple(bigram.shape)} {bigram.dtype} beside an embedding "
                          f"{tuple(table.shape)} {table.dtype}")
    _guard("core", "elementwise", table.device, n_slots=prev.shape[0])
    _check(_fn("core", "mv_embed_bigram")(
        _need(table, "embedding table"), _need(bigram, "bigram table"), _dt(table), _need(tokens, "tokens", torch.int32),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32), _need(cu, "cu", torch.int32),
        _need(slots, "slots", torch.int32), _need(prev, "previous tokens", torch.int32),
        _need(out, "embedding out", torch.float32, (N, H)), _need(kept, "embedding copy", torch.float32, (N, H), True),
        N, H, bigram.shape[0] - 1, int(mul_prev), int(mul_cur), _stream()), "mv_embed_bigram")
    account(N * H * (2 * table.element_size() + (8 if kept is not None else 4)))
    return out


def add_rows_vector(x: torch.Tensor, rows: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> torch.Tensor:
    """x[n] += rows[n] + vec, all float32 (either may be None)."""
    N, H = x.shape
    _check(_fn("core", "mv_add_rows_vector")(
        _need(x, "stream", torch.float32), _need(rows, "rows", torch.float32, (N, H), True),
        _need(vec, "vector", torch.float32, (H,), True), N, H, _stream()), "mv_add_rows_vector")
    account(N * H * (12 if rows is not None else 8))
    return x


def _check_latent_pool(pool: torch.Tensor, page_size: int, width: int, what: str) -> None:
    if pool.dim() != 2 or pool.shape[1] != page_size * width or not pool.is_cuda or pool.stride(1) != 1:
        raise KernelError(f"{what}: cache pool shape {tuple(pool.shape)}, expected [pages, {page_size} rows x {width}]")
    if page_size & (page_size - 1):
        raise KernelError(f"{what}: page size {page_size} is not a power of two")


LATENT_MAX_RANK = 1024
LATENT_MAX_ROT = 512


def latent_prepare(proj: torch.Tensor, q0: int, c0: int, w_c: torch.Tensor, eps: float, inv_freq: Optional[torch.Tensor],
                   positions, seq_of, page_table, pool: torch.Tensor, page_size: int, qa: torch.Tensor, nh: int, dim: int,
                   rot: int, rank: int, rot_dims: Optional[int] = None) -> None:
    """From float32 rows of a fused projection (q at column ``q0``: per head [dim | rot]; the latent at column ``c0``:
    [rank | rot]): the latent's first ``rank`` numbers over their root mean square times ``w_c``, its last ``rot`` and
    every head's last ``rot`` of q rotated (their first ``rot_dims``, all by default: element i with i + rot_dims / 2,
    angle pos * inv_freq[i]; the others pass unchanged); the row [rank + rot]
    goes into the token's place of its page, the rotated parts of q into the last ``rot`` columns of ``qa``
    [N, nh, rank + rot] (float32; None: the queries are prepared elsewhere)."""
    N = proj.shape[0]
    if (not proj.is_cuda or proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1
            or q0 < 0 or q0 + nh * (dim + rot) > proj.shape[1] or c0 < 0 or c0 + rank + rot > proj.shape[1]):
        raise KernelError(f"latent_prepare: projection {proj.dtype} {tuple(proj.shape)} does not hold q at {q0} and the "
                          f"latent at {c0} for {N} rows")
    rot_dims = rot if rot_dims is None else int(rot_dims)
    if rot_dims % 2 or not 0 <= rot_dims <= rot <= LATENT_MAX_ROT or not 1 <= rank <= LATENT_MAX_RANK:
        raise KernelError(f"latent_prepare: rank {rank} (1..{LATENT_MAX_RANK}), {rot_dims} of {rot} (<= {LATENT_MAX_ROT}) "
                          f"elements rotated (an even number)")
    _check_latent_pool(pool, page_size, rank + rot, "latent_prepare")
    _guard("core", "latent_attention", proj.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_latent_prepare")(
        proj.data_ptr(), proj.stride(0), int(q0), int(c0), _need(w_c, "latent norm weight", torch.float32, (rank,)),
        float(eps), _need(inv_freq, "inv_freq", torch.float32, (rot_dims // 2,), rot_dims == 0),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(page_table, "page table", torch.int32), page_table.shape[1], int(page_size), pool.data_ptr(), pool.stride(0),
        _dt(pool), _need(qa, "absorbed q", torch.float32, (N, nh, rank + rot), True), N, nh, dim, rot, rank, rot_dims, _stream()),
        "mv_latent_prepare")
    account(N * (nh * rot * 8 + (rank + rot) * (4 + pool.element_size())))


def head_product(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, nh: int, n_in: int, n_out: int, *,
                 transposed: bool = False, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One small matrix per head: y[n, h, :n_out] = W_h x[n, h, :n_in] with ``w`` [nh * n_out, n_in], or with
    ``transposed`` W_h^T x with ``w`` [nh * n_in, n_out].  ``x`` float32 [N, nh, >= n_in] and ``y`` [N, nh, >= n_out]
    (float32 or the model's dtype) may be views with any row and head strides.  ``gate``: float32 logits
    [N, nh * n_out] (a column slice is fine); the result is multiplied by sigmoid(gate)."""
    N = x.shape[0]
    for t, what, width in ((x, "input", n_in), (y, "output", n_out)):
        if not t.is_cuda or t.dim() != 3 or t.shape[0] != N or t.shape[1] != nh or t.shape[2] < width or t.stride(2) != 1:
            raise KernelError(f"head_product: {what} {tuple(t.shape)} strides {t.stride()} for {N} rows, {nh} heads of {width}")
    if x.dtype != torch.float32:
        raise KernelError(f"head_product: input is {x.dtype}, expected float32")
    rows, cols = (nh * n_in, n_out) if transposed else (nh * n_out, n_in)
    gp, ldg = _cols(gate, "head_product gate", N, nh * n_out) if gate is not None else (None, 0)
    _check(_fn("core", "mv_head_product")(
        x.data_ptr(), x.stride(0), x.stride(1), _need(w, "head matrices", None, (rows, cols)), _dt(w), int(bool(transposed)),
        gp, ldg, y.data_ptr(), _dt(y), y.stride(0), y.stride(1), N, nh, int(n_in), int(n_out), _stream()), "mv_head_product")
    account(w.numel() * w.element_size() + N * nh * (n_in * 4 + n_out * y.element_size()), 2 * N * nh * n_in * n_out)
    return y


# a (token, head tile) whose keys would keep one block busy for more than this many of them is cut into shares
LATENT_SPLIT_KEYS = 128
LATENT_MAX_SPLITS = 32


def latent_splits(n_tokens: int, n_heads: int, longest: int, sm_count: int) -> int:
    """Into how many shares of the keys a step of ``n_tokens`` query tokens is cut: enough blocks to fill the device
    twice, no share under ``LATENT_SPLIT_KEYS`` keys."""
    blocks = max(1, n_tokens * ((n_heads + 7) // 8))
    want = (2 * sm_count + blocks - 1) // blocks
    return int(max(1, min(want, longest // LATENT_SPLIT_KEYS, LATENT_MAX_SPLITS)))


def latent_attention(qa: torch.Tensor, pool: torch.Tensor, page_size: int, page_table, positions, seq_of,
                     out: torch.Tensor, nh: int, rank: int, rot: int, scale: float, *, window: int = 0,
                     sinks: Optional[torch.Tensor] = None, splits: int = 1,
                     part: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """Causal softmax attention of every token of the step over its sequence's cached rows [rank + rot] (which already
    hold the step's own): all heads read the same rows as keys, and the rows' first ``rank`` numbers as values.
    ``qa`` float32 [N, nh, rank + rot], ``out`` float32 [N, nh, rank].  ``window`` w > 0: query i reads key j if
    0 <= i - j < w.  ``sinks`` [nh]: exp(sink) joins each head's denominator.  Scores and softmax are float32.
    ``splits`` > 1: the keys of every token are cut into that many shares, one block each, and a second kernel puts
    the shares together; ``part`` = (float32 [N, nh, splits, rank], float32 [N, nh, splits, 2]) is their scratch."""
    N = qa.shape[0]
    if not 1 <= rank <= LATENT_MAX_RANK or rot < 0:
        raise KernelError(f"latent_attention: rank {rank} must lie in 1..{LATENT_MAX_RANK}")
    _check_latent_pool(pool, page_size, rank + rot, "latent_attention")
    splits = int(splits)
    if splits > 1 and part is None:
        raise KernelError("latent_attention: shares of the keys need their scratch")
    _guard("core", "latent_attention", qa.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_latent_attention")(
        _need(qa, "absorbed q", torch.float32, (N, nh, rank + rot)), pool.data_ptr(), pool.stride(0), _dt(pool),
        _need(page_table, "page table", torch.int32), page_table.shape[1], int(page_size),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(sinks, "sinks", torch.float32, (nh,), True), _need(out, "attention out", torch.float32, (N, nh, rank)),
        N, nh, rank, rot, float(scale), int(window), splits,
        _need(part[0], "shares", torch.float32, (N, nh, splits, rank)) if splits > 1 else None,
        _need(part[1], "shares' sums", torch.float32, (N, nh, splits, 2)) if splits > 1 else None,
        _stream()), "mv_latent_attention")
    return out


def latent_prefill_fits(dim: int, rot: int, dv: int, rank: int) -> bool:
    """Whether the tensor-core kernels for steps of many tokens take these sizes."""
    return dim % 8 == 0 and rot % 8 == 0 and (dim + rot) % 16 == 0 and 16 <= dim + rot <= 192 and dv % 16 == 0 \
        and 16 <= dv <= 128 and rank % 8 == 0


def latent_query(proj: torch.Tensor, q0: int, inv_freq: Optional[torch.Tensor], positions, q: torch.Tensor, nh: int,
                 dim: int, rot: int, rot_dims: int) -> torch.Tensor:
    """``q`` [N, nh, dim + rot] (bfloat16) from float32 rows of a projection (the queries from column ``q0``), the first
    ``rot_dims`` of every head's last ``rot`` elements turned (i with i + rot_dims / 2, angle pos * inv_freq[i])."""
    N = q.shape[0]
    if (not proj.is_cuda or proj.dtype != torch.float32 or proj.dim() != 2 or proj.shape[0] != N or proj.stride(1) != 1
            or q0 < 0 or q0 + nh * (dim + rot) > proj.shape[1] or rot_dims % 2 or not 0 <= rot_dims <= rot):
        raise KernelError(f"latent_query: projection {proj.dtype} {tuple(proj.shape)} does not hold {nh} heads of "
                          f"{dim} + {rot} at {q0} for {N} rows")
    _check(_fn("bf16", "mv_latent_query")(
        proj.data_ptr(), proj.stride(0), int(q0), _need(inv_freq, "inv_freq", torch.float32, (rot_dims // 2,), rot_dims == 0),
        _need(positions, "positions", torch.int32), _need(q, "q", torch.bfloat16, (N, nh, dim + rot)), N, nh, dim, rot,
        int(rot_dims), _stream()), "mv_latent_query")
    account(N * nh * (dim + rot) * 6)
    return q


def latent_gather(pool: torch.Tensor, page_size: int, page_table, cu, starts, n_seqs: int, window: int,
                  c: torch.Tensor, r: torch.Tensor) -> None:
    """The cached rows [rank | rot] that the step's tokens can see (sequence b's positions from
    max(0, starts[b] - window + 1), from 0 without a window, to its last), sequence after sequence, into ``c``
    [rows, rank] and ``r`` [rows, rot], bfloat16."""
    rows, rank, rot = c.shape[0], c.shape[1], r.shape[1]
    _check_latent_pool(pool, page_size, rank + rot, "latent_gather")
    if pool.dtype != torch.bfloat16:
        raise KernelError(f"latent_gather: the cache is {pool.dtype}, expected bfloat16")
    _guard("bf16", "latent_attention_prefill", pool.device, n_pages=pool.shape[0])
    _check(_fn("bf16", "mv_latent_gather")(
        pool.data_ptr(), pool.stride(0), _need(page_table, "page table", torch.int32), page_table.shape[1], int(page_size),
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32), int(n_seqs), int(window), rank, rot,
        _need(c, "latents", torch.bfloat16, (rows, rank)), _need(r, "rotated keys", torch.bfloat16, (rows, rot)), rows,
        _stream()), "mv_latent_gather")
    account(rows * (rank + rot) * 4)


def latent_attention_prefill(q: torch.Tensor, kx: torch.Tensor, v0: int, r: torch.Tensor, cu, starts, n_seqs: int,
                             out: torch.Tensor, nh: int, dim: int, rot: int, dv: int, scale: float, *, window: int = 0,
                             sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal softmax attention on the tensor cores for steps of many tokens: ``q`` [N, nh, dim + rot] against the
    gathered rows' keys and values ``kx`` [rows, >= v0 + nh dv] (head h's unrotated key at column h dim, its value at
    v0 + h dv) and the shared rotated key part ``r`` [rows, rot]; all bfloat16, scores and softmax float32.
    ``gate``: float32 logits [N, nh dv] (a column slice is fine); ``out`` [N, nh dv] is multiplied by their sigmoid."""
    N, rows = q.shape[0], kx.shape[0]
    if not latent_prefill_fits(dim, rot, dv, 8):
        raise KernelError(f"latent_attention_prefill: sizes {dim} + {rot}, {dv} are not served")
    if kx.dtype != torch.bfloat16 or kx.dim() != 2 or kx.stride(1) != 1 or kx.shape[1] < v0 + nh * dv or v0 < nh * dim:
        raise KernelError(f"latent_attention_prefill: keys and values {kx.dtype} {tuple(kx.shape)}, values from {v0}")
    gp, ldg = _cols(gate, "latent_attention_prefill gate", N, nh * dv) if gate is not None else (None, 0)
    _check(_fn("bf16", "mv_latent_attention_prefill")(
        _need(q, "q", torch.bfloat16, (N, nh, dim + rot)), kx.data_ptr(), kx.stride(0), int(v0),
        _need(r, "rotated keys", torch.bfloat16, (rows, rot)), _need(cu, "cu", torch.int32),
        _need(starts, "starts", torch.int32), _need(sinks, "sinks", torch.float32, (nh,), True), gp, ldg,
        _need(out, "attention out", torch.bfloat16, (N, nh * dv)), N, int(n_seqs), nh, dim, rot, dv, float(scale),
        int(window), _stream()), "mv_latent_attention_prefill")
    return out


# steps that bring a sequence this many tokens or more run the recurrence from rows prepared by a kernel before it
DELTA_LONG_STEP = 8


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, a: torch.Tensor,
               dt_bias: torch.Tensor, a_log: torch.Tensor, state: torch.Tensor, slots, cu, out: torch.Tensor,
               n_seqs: int, n_heads: int, kv_heads: int, dk: int, dv: int, *, q_scale: float,
               norm_eps: float = 1e-6, max_len: int = 1, ws=None, head_decay: bool = False) -> torch.Tensor:
    """The gated delta rule with a decay per key channel, token by token: per head S <- diag(g) S;
    u = sigmoid(beta) (v - S^T k); S <- S + k u^T; o = S^T q, with q and k made unit vectors per head first
    (x / sqrt(sum x^2 + norm_eps), q also times ``q_scale``) and g = exp(-exp(a_log_h) softplus(a + dt_bias)).
    q, k [N, kv_heads * dk] (head h reads head h // (n_heads / kv_heads)), v [N, n_heads * dv], beta [N, n_heads],
    a [N, n_heads * dk] (with ``head_decay`` one decay a head: a [N, n_heads], dt_bias [n_heads]): float32, column
    slices are fine; ``state`` float32 [slots, n_heads, dv, dk]; ``out``
    float32 [N, n_heads * dv].  ``max_len``: the most tokens that a sequence brings; from ``DELTA_LONG_STEP`` on
    (and with a workspace ``ws`` for the prepared rows) unit vectors, decays and beta are worked out once a token by
    a kernel of their own and the walk along the sequence holds the recurrence alone."""
    N = out.shape[0]
    if not 1 <= dk <= MAX_SCAN_KEY_DIM or kv_heads < 1 or n_heads % kv_heads:
        raise KernelError(f"delta_scan: key size {dk} (1..{MAX_SCAN_KEY_DIM}), {n_heads} heads on {kv_heads} kv heads")
    long_step = ws is not None and max_len >= DELTA_LONG_STEP
    qp, ldq = _cols(q, "delta_scan q", N, kv_heads * dk)
    kp, ldk = _cols(k, "delta_scan k", N, kv_heads * dk)
    vp, ldv = _cols(v, "delta_scan v", N, n_heads * dv)
    bp, ldb = _cols(beta, "delta_scan beta", N, n_heads)
    n_decays = n_heads if head_decay else n_heads * dk
    ap, lda = _cols(a, "delta_scan decay", N, n_decays)
    _guard("core", "delta_rule", out.device, n_slots=state.shape[0])
    if long_step:
        # a row: q and k of the q/k heads, the decays, beta, k . q; padded to 16 bytes (as the kernel lays it out)
        width = (2 * kv_heads * dk + n_heads * dk + n_heads + kv_heads + 3) & ~3
        prep = ws.get("delta_scan.prep", (N, width), torch.float32)
        _check(_fn("core", "mv_delta_scan_long")(
            qp, ldq, kp, ldk, vp, ldv, bp, ldb, ap, lda, _need(dt_bias, "dt_bias", torch.float32, (n_decays,)),
            _need(a_log, "A_log", torch.float32, (n_heads,)), float(q_scale), float(norm_eps), prep.data_ptr(),
            _need(state, "delta_scan state", torch.float32, (None, n_heads, dv, dk)), _need(slots, "slots", torch.int32),
            _need(cu, "cu", torch.int32), _need(out, "delta_scan out", torch.float32, (N, n_heads * dv)), N, int(n_seqs),
            n_heads, kv_heads, dk, dv, int(bool(head_decay)), _stream()), "mv_delta_scan_long")
        account(2 * n_seqs * n_heads * dv * dk * 4 + N * (2 * kv_heads * dk + n_heads * (2 * dv + dk + 1)) * 4
                + 2 * prep.numel() * 4, 6 * N * n_heads * dk * dv)
        return out
    _check(_fn("core", "mv_delta_scan")(
        qp, ldq, kp, ldk, vp, ldv, bp, ldb, ap, lda, _need(dt_bias, "dt_bias", torch.float32, (n_decays,)),
        _need(a_log, "A_log", torch.float32, (n_heads,)), float(q_scale), float(norm_eps),
        _need(state, "delta_scan state", torch.float32, (None, n_heads, dv, dk)), _need(slots, "slots", torch.int32),
        _need(cu, "cu", torch.int32), _need(out, "delta_scan out", torch.float32, (N, n_heads * dv)), int(n_seqs), n_heads,
        kv_heads, dk, dv, int(bool(head_decay)), _stream()), "mv_delta_scan")
    account(2 * n_seqs * n_heads * dv * dk * 4 + N * (2 * kv_heads * dk + n_heads * (2 * dv + dk + 1)) * 4,
            6 * N * n_heads * dk * dv)
    return out


SWIGLU_GROUP = 16


def swiglu(gu: torch.Tensor, out: torch.Tensor, group: int = 0) -> torch.Tensor:
    """out[n, f] = silu(gate) * up.  ``group`` 0: gate and up are the two halves
    of a row of ``gu``; 16: they alternate in groups of 16 columns."""
    N, F2 = gu.shape
    F = F2 // 2
    if group and F % group:
        raise KernelError(f"swiglu: width {F} is not a multiple of the group size {group}")
    _check(_fn("core", "mv_swiglu")(
        _need(gu, "swiglu in", torch.float32), _need(out, "swiglu out", None, (N, F)), _dt(out), N, F, int(group),
        _stream()), "mv_swiglu")
    account(_nbytes(gu, out))
    return out


STORE, ACCUMULATE = "store", "accumulate"


def _account_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
    if _profile is not None:
        account(_nbytes(x, w) + (2 if accumulate else 1) * out.numel() * out.element_size(),
                2 * x.shape[0] * w.shape[0] * w.shape[1])


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
              accumulate: bool = False) -> torch.Tensor:
    """out = x @ w.T (+ bias), or out += ... when ``accumulate`` (out float32).
    CUDA-core kernel, float32 accumulation, any sizes."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != w.dtype:
        raise KernelError(f"gemm: x is {x.dtype} but w is {w.dtype}")
    if accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    _check(_fn("core", "mv_gemm_simt")(
        _need(x, "gemm x"), _need(w, "gemm w"), _dt(x), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, N, _stream()), "mv_gemm_simt")
    _account_gemm(x, w, out, accumulate)
    return out


SMALL_M_MAX = 64




@dataclass
class NormLink:
    """A norm carried by the two products around it, in a step of few tokens.  The product
    that completes the residual stream (``emit``) also writes ``xg`` = bf16(x_new * weight)
    and, per tile of its rows, the sum of x_new^2 into ``partials``; the product that reads
    the normed rows (``scale``) takes ``xg`` as its input and multiplies every token's
    results by rsqrt(sum(partials) / dim + eps).  Statistics and scale are float32."""
    norm: object                   # the norm part this stands for (identity only)
    weight: torch.Tensor           # float32 [dim]
    eps: float
    dim: int
    xg: torch.Tensor               # bfloat16 [tokens, dim]
    partials: torch.Tensor         # float32 [tokens, >= ceil(dim / 16)]: the tile sums of one token lie together
    n_partials: int = 0            # set by the emitting product


def gemm_small_m_tile_rows(N: int, mode: int) -> int:
    return int(_fn("bf16", "mv_gemm_small_m_tile_rows")(int(N), int(mode)))


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False, swiglu: bool = False, scale: Optional[NormLink] = None,
                 emit: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """out = x @ w.T for at most 64 rows of x, bfloat16 operands: the
    weight-streaming tensor-core kernel of the decode step.  ``scale`` / ``emit``: the
    two ends of a :class:`NormLink`.  ``ahead``: (address, bytes) of what the step's next
    product will read; the kernel asks the L2 cache for it once it has its own weights."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8:
        raise KernelError(f"gemm_small_m: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_small_m: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    link = _link_args(x, M, N, K, mode, scale, emit, -(-N // gemm_small_m_tile_rows(N, 2)))
    _check(_fn("bf16", "mv_gemm_small_m")(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link, *(ahead or (None, 0)), _stream()), "mv_gemm_small_m")
    _account_gemm(x, w, out, accumulate)
    return out


SHORTCONV_FUSED_MAX_ROWS = 8


def gemm_small_m_shortconv(x: torch.Tensor, w_in: torch.Tensor, b_in: Optional[torch.Tensor], taps: torch.Tensor,
                           b_conv: Optional[torch.Tensor], state: torch.Tensor, slots: torch.Tensor,
                           out: torch.Tensor, *, scale: Optional[NormLink] = None,
                           ahead: Optional[tuple] = None) -> torch.Tensor:
    """A decode step's gated short convolution together with its input projection, in one kernel:
    [B | C | x] = x @ w_in.T (+ b_in), out = C * conv(B * x) with the sequences' kept values in
    ``state`` [n_slots, k-1, H], which it shifts and updates for the rows' sequences (``slots[m]`` is
    row m's).  At most 8 rows, one a sequence; bfloat16 operands; ``scale`` and ``ahead`` as in
    ``gemm_small_m``."""
    M, K = x.shape
    H, k = taps.shape
    if tuple(w_in.shape) != (3 * H, K):
        raise KernelError(f"shortconv: in_proj weight is {tuple(w_in.shape)}, expected [{3 * H}, {K}]")
    if x.dtype != torch.bfloat16 or w_in.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m_shortconv: operands must be bfloat16, got {x.dtype} and {w_in.dtype}")
    if not 1 <= M <= SHORTCONV_FUSED_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_small_m_shortconv: needs 1..{SHORTCONV_FUSED_MAX_ROWS} rows and K a multiple "
                          f"of 8, got M={M}, K={K}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    if slots.numel() < M:
        raise KernelError(f"shortconv: {slots.numel()} slots for {M} rows")
    sp, n_sp, s_stride, dim, eps = _link_args(x, M, 3 * H, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_small_m_shortconv")(
        _need(x, "gemm x"), _need(w_in, "gemm w"), _need(b_in, "in_proj bias", torch.float32, (3 * H,), True),
        _need(taps, "shortconv taps", torch.float32), _need(b_conv, "shortconv bias", torch.float32, (H,), True),
        state.data_ptr(), _need(slots, "slots", torch.int32), _need(out, "shortconv out", torch.bfloat16, (M, H)),
        M, H, K, k, sp, n_sp, s_stride, dim, eps, *(ahead or (None, 0)), _stream()), "mv_gemm_small_m_shortconv")
    _account_gemm(x, w_in, out, False)
    return out


HEADS_FUSED_HEAD_DIM = 64


def gemm_small_m_heads(x: torch.Tensor, w_qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                       eps: float, inv_freq: Optional[torch.Tensor], half_split: bool, positions, seq_of,
                       page_table, pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, *,
                       scale: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """The fused q/k/v projection together with what ``qk_prepare`` does, in one kernel, for steps of
    at most 8 tokens, heads of 64 and a bfloat16 cache: q comes out normed and rotated in ``q_out``,
    k (normed, rotated) and v go into the tokens' rows of the paged cache.  ``scale`` and ``ahead``
    as in ``gemm_small_m``."""
    M, K = x.shape
    hd = HEADS_FUSED_HEAD_DIM
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K):
        raise KernelError(f"gemm_small_m_heads: weight is {tuple(w_qkv.shape)}, expected "
                          f"[{(nh + 2 * nkv) * hd}, {K}] ({nh} + 2 x {nkv} heads of {hd})")
    if x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m_heads: operands and cache must be bfloat16, got {x.dtype}, "
                          f"{w_qkv.dtype} and {pool.dtype}")
    if not 1 <= M <= SHORTCONV_FUSED_MAX_ROWS or K % 8:
        raise KernelError(f"gemm_small_m_heads: needs 1..{SHORTCONV_FUSED_MAX_ROWS} rows and K a multiple "
                          f"of 8, got M={M}, K={K}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "gemm_small_m_heads")
    _need(page_table, "page table", torch.int32)
    sp, n_sp, s_stride, dim, eps_norm = _link_args(x, M, (nh + 2 * nkv) * hd, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_small_m_heads")(
        _need(x, "gemm x"), _need(w_qkv, "gemm w"), _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"), pool.stride(0),
        _need(q_out, "q out", torch.bfloat16, (M, nh * hd)), M, nh, nkv, K, sp, n_sp, s_stride, dim, eps_norm,
        *(ahead or (None, 0)), _stream()), "mv_gemm_small_m_heads")
    _account_gemm(x, w_qkv, q_out, False)
    return q_out


def _link_args(x, M: int, N: int, K: int, mode: int, scale: Optional[NormLink], emit: Optional[NormLink],
               tiles: int):
    """The nine arguments that carry a norm through a product: (partials, count, stride, dim, eps)
    of the link it consumes and (weight, rows, partials, stride) of the link it emits, which
    writes ``tiles`` sums a row."""
    sp, n_sp, s_stride, dim, eps, eg, ex, ep, e_stride = None, 0, 0, 0, 0.0, None, None, None, 0
    if scale is not None:
        if scale.n_partials <= 0 or scale.dim != K or x.data_ptr() != scale.xg.data_ptr():
            raise KernelError("gemm: the scaled input must be the rows that the norm link's producer wrote")
        _need(scale.partials, "norm partials", torch.float32)
        sp, n_sp, s_stride = scale.partials.data_ptr(), scale.n_partials, scale.partials.shape[1]
        dim, eps = scale.dim, float(scale.eps)
    if emit is not None:
        if mode != 2 or emit.dim != N:
            raise KernelError("gemm: only a product that adds into the residual stream can emit a norm")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        _need(emit.xg, "normed rows", torch.bfloat16, (M, N))
        _need(emit.partials, "norm partials", torch.float32)
        if emit.partials.dim() != 2 or emit.partials.shape[0] < M or emit.partials.shape[1] < tiles:
            raise KernelError(f"gemm: norm partials [{tuple(emit.partials.shape)}] cannot hold {tiles} tile "
                              f"sums for each of {M} rows")
        eg, ex, ep, e_stride = emit.weight.data_ptr(), emit.xg.data_ptr(), emit.partials.data_ptr(), emit.partials.shape[1]
        emit.n_partials = tiles
    return sp, n_sp, s_stride, dim, eps, eg, ex, ep, e_stride


_error_flags = {}
_error_mirrors = {}
_ERROR_ROLES = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue", 4: "a guarded index"}


def _error_flag(device) -> torch.Tensor:
    """One int per device that a kernel sets when one of its bounded waits ran out (or, in a build
    with index checks, when an index lay outside its bounds)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def _error_text(key: int, code: int) -> str:
    role = _ERROR_ROLES.get(code, f"code {code}")
    if code == 4:
        return (f"a kernel on cuda:{key} was handed an index outside its bounds (a page or a slot); it skipped "
                f"the access and its output is not valid")
    return (f"a tensor-core kernel on cuda:{key} gave up waiting on a barrier in {role}; "
            f"its output is not valid")


def note_device_errors(device) -> None:
    """Enqueue a copy of the device's error flag into pinned host memory, on the current stream
    (may be recorded into a CUDA graph).  ``raise_seen_device_errors`` looks at that copy."""
    key = torch.device(device).index or 0
    mirror = _error_mirrors.get(key)
    if mirror is None:
        mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        _error_mirrors[key] = mirror
    code = _fn("core", "mv_copy_to_host")(mirror.data_ptr(), _error_flag(device).data_ptr(), 4, _stream())
    if code != 0:
        raise KernelError(f"copying the error flag to the host failed with CUDA error {code}")


def raise_seen_device_errors(device) -> None:
    """Raise if a copy of the error flag that has arrived on the host is set; does not wait for the
    device.  Exact where the host has just waited for work enqueued after ``note_device_errors``."""
    key = torch.device(device).index or 0
    mirror = _error_mirrors.get(key)
    if mirror is None:
        return
    code = int(mirror[0])
    if code:
        torch.cuda.synchronize(device)
        _error_flags[key].zero_()
        torch.cuda.synchronize(device)
        mirror.zero_()
        raise KernelError(_error_text(key, code))


def raise_device_error(device, code: int) -> None:
    """A kernel's fault arrived on the host by another way than the mirror (with the sampled tokens):
    clear the flag and raise."""
    key = torch.device(device).index or 0
    torch.cuda.synchronize(device)
    _error_flag(device).zero_()
    torch.cuda.synchronize(device)
    if key in _error_mirrors:
        _error_mirrors[key].zero_()
    raise KernelError(_error_text(key, int(code)))


def check_device_errors() -> None:
    """Raise if a kernel reported a fault (synchronises the device)."""
    for key, flag in _error_flags.items():
        code = int(flag.item())
        if code:
            flag.zero_()
            if key in _error_mirrors:
                torch.cuda.synchronize(flag.device)
                _error_mirrors[key].zero_()
            raise KernelError(_error_text(key, code))


_PREFILL_GEMM = os.environ.get("MIVI_PREFILL_GEMM", "auto")      # pair | single | auto


def gemm_tc_pair_takes(M: int, N: int) -> bool:
    """Shapes for which two multiprocessors share a 256 x 256 tile (``gemm_tc_pair.cu``): more than
    128 rows, and enough tiles that most pairs of the device get one."""
    if _PREFILL_GEMM == "single" or M <= 128 or N < 128:
        return False
    tiles = -(-M // 256) * -(-N // 256)
    return _PREFILL_GEMM == "pair" or tiles >= 48 * n_sms() // 148


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, swiglu: bool = False, pair: Optional[bool] = None,
            scale: Optional[NormLink] = None, emit: Optional[NormLink] = None) -> torch.Tensor:
    """out = x @ w.T, bfloat16 operands, on the tcgen05 tensor cores (TMA
    loads, accumulator in tensor memory): the matrix product of prefill.
    ``pair``: True: the kernel in which two multiprocessors share a 256 x 256 tile, False: the
    one-multiprocessor kernels, None: by shape (``gemm_tc_pair_takes``).  ``scale`` / ``emit``: the two
    ends of a :class:`NormLink`; every kernel here applies a scale, only the pair kernel emits (N in
    steps of 32)."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if K % 8 or K < 8:
        raise KernelError(f"gemm_tc: K must be a multiple of 8 (16-byte rows for TMA), got {K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_tc: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    if pair is None:
        pair = gemm_tc_pair_takes(M, N) or (emit is not None and M > 128 and N >= 128)
    elif pair and (M <= 128 or N < 128):
        raise KernelError(f"gemm_tc: the pair kernel needs more than 128 rows and at least 128 columns, got {M} x {N}")
    if pair:
        if emit is not None and N % 32:
            raise KernelError(f"gemm_tc: a product that emits a norm needs N in steps of 32, got {N}")
        link = _link_args(x, M, N, K, mode, scale, emit, -(-N // 256))
        _check(_fn("bf16", "mv_gemm_tc_pair")(
            _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
            out.data_ptr(), mode, M, N, K, ldo, *link, _error_flag(x.device).data_ptr(), _stream()), "mv_gemm_tc_pair")
        _account_gemm(x, w, out, accumulate)
        return out
    if emit is not None:
        raise KernelError("gemm_tc: only the kernel of two multiprocessors a tile emits a norm")
    link = _link_args(x, M, N, K, mode, scale, None, 0)
    entry = "mv_gemm_tc"
    _check(_fn("bf16", entry)(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link[:5], _error_flag(x.device).data_ptr(), _stream()), entry)
    _account_gemm(x, w, out, accumulate)
    return out


def gemm_tc_swap(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False, swiglu: bool = False, scale: Optional[NormLink] = None,
                 emit: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """out = x @ w.T on the tcgen05 tensor cores with the operands' roles swapped (rows of w
    on the MMA's M side, up to 256 tokens a tile on its N side): a TMA pipeline that streams w
    once, K cut over the blocks of a cluster.  Same contract as ``gemm_small_m``, for any number of
    rows: the kernel of steps whose cost is reading the weights."""
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x is [{M}, {K}] but w is [{N}, {K2}]")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap: operands must be bfloat16, got {x.dtype} and {w.dtype}")
    if M < 1 or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap: needs at least one row and K a multiple of 8, got M={M}, K={K}")
    ldo = N
    if swiglu:
        if N % 32:
            raise KernelError(f"gemm_tc_swap: the SwiGLU epilogue needs rows in groups of 32, got {N}")
        mode, ldo = 3, N // 2
        _need(out, "gemm out", torch.bfloat16, (M, N // 2))
    elif accumulate:
        mode = 2
        _need(out, "gemm out", torch.float32, (M, N))
    else:
        mode = 0 if out.dtype == torch.float32 else 1
        _need(out, "gemm out", None, (M, N))
        _dt(out)
    link = _link_args(x, M, N, K, mode, scale, emit, -(-N // 128))
    _check(_fn("bf16", "mv_gemm_tc_swap")(
        _need(x, "gemm x"), _need(w, "gemm w"), _need(bias, "gemm bias", torch.float32, (N,), True),
        out.data_ptr(), mode, M, N, K, ldo, *link, *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()),
        "mv_gemm_tc_swap")
    _account_gemm(x, w, out, accumulate)
    return out


def gemm_tc_swap_shortconv(x: torch.Tensor, w_in: torch.Tensor, b_in: Optional[torch.Tensor], taps: torch.Tensor,
                           b_conv: Optional[torch.Tensor], state: torch.Tensor, slots: torch.Tensor,
                           out: torch.Tensor, *, scale: Optional[NormLink] = None,
                           ahead: Optional[tuple] = None) -> torch.Tensor:
    """``gemm_small_m_shortconv`` for up to 64 rows, on the tcgen05 kernel with swapped operands.  The rows
    of ``w_in`` come regrouped by :func:`group_conv_rows` (32 channels' B, C and x rows together; the width a
    multiple of 32), so that a block's one tile holds all three of its channels."""
    M, K = x.shape
    H, k = taps.shape
    if H % CONV_ROW_GROUP:
        raise KernelError(f"shortconv: regrouped rows need a width in steps of {CONV_ROW_GROUP}, got {H}")
    if tuple(w_in.shape) != (3 * H, K):
        raise KernelError(f"shortconv: in_proj weight is {tuple(w_in.shape)}, expected [{3 * H}, {K}]")
    if x.dtype != torch.bfloat16 or w_in.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap_shortconv: operands must be bfloat16, got {x.dtype} and {w_in.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap_shortconv: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    if slots.numel() < M:
        raise KernelError(f"shortconv: {slots.numel()} slots for {M} rows")
    sp, n_sp, s_stride, dim, eps = _link_args(x, M, 3 * H, K, 1, scale, None, 0)[:5]
    entry = "mv_gemm_tc_swap_shortconv"
    _check(_fn("bf16", entry)(
        _need(x, "gemm x"), _need(w_in, "gemm w"), _need(b_in, "in_proj bias", torch.float32, (3 * H,), True),
        _need(taps, "shortconv taps", torch.float32), _need(b_conv, "shortconv bias", torch.float32, (H,), True),
        state.data_ptr(), _need(slots, "slots", torch.int32), _need(out, "shortconv out", torch.bfloat16, (M, H)),
        M, H, K, k, sp, n_sp, s_stride, dim, eps, *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()),
        entry)
    _account_gemm(x, w_in, out, False)
    return out


CONV_ROW_GROUP = 32


def group_conv_rows(w_in: torch.Tensor) -> torch.Tensor:
    """The rows of a short convolution's input projection [3 H, K] (B rows, C rows, x rows) regrouped for
    ``gemm_tc_swap_shortconv``: the B rows of channels 0..31, their C rows, their x rows, then
    the same of channels 32..63, and so on.  A copy; H a multiple of 32."""
    H3, K = w_in.shape
    H = H3 // 3
    if H3 != 3 * H or H % CONV_ROW_GROUP:
        raise KernelError(f"shortconv: cannot regroup the rows of a [{H3}, {K}] projection by {CONV_ROW_GROUP} channels")
    g = CONV_ROW_GROUP
    return w_in.view(3, H // g, g, K).permute(1, 0, 2, 3).reshape(H3, K).contiguous()


def gemm_tc_swap_heads(x: torch.Tensor, w_qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor],
                       eps: float, inv_freq: Optional[torch.Tensor], positions, seq_of, page_table,
                       pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, *,
                       scale: Optional[NormLink] = None, ahead: Optional[tuple] = None) -> torch.Tensor:
    """``gemm_small_m_heads`` for up to 64 tokens, on the tcgen05 kernel with swapped operands (heads of 64,
    the pairs (2i, 2i+1) only): a tile of 128 rows is two heads, a half-warp finishes one for a token."""
    M, K = x.shape
    hd = HEADS_FUSED_HEAD_DIM
    if tuple(w_qkv.shape) != ((nh + 2 * nkv) * hd, K):
        raise KernelError(f"gemm_tc_swap_heads: weight is {tuple(w_qkv.shape)}, expected "
                          f"[{(nh + 2 * nkv) * hd}, {K}] ({nh} + 2 x {nkv} heads of {hd})")
    if x.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc_swap_heads: operands and cache must be bfloat16, got {x.dtype}, "
                          f"{w_qkv.dtype} and {pool.dtype}")
    if not 1 <= M <= SMALL_M_MAX or K % 8 or K < 8:
        raise KernelError(f"gemm_tc_swap_heads: needs 1..{SMALL_M_MAX} rows and K a multiple of 8, got M={M}, K={K}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "gemm_tc_swap_heads")
    _need(page_table, "page table", torch.int32)
    sp, n_sp, s_stride, dim, eps_norm = _link_args(x, M, (nh + 2 * nkv) * hd, K, 1, scale, None, 0)[:5]
    _check(_fn("bf16", "mv_gemm_tc_swap_heads")(
        _need(x, "gemm x"), _need(w_qkv, "gemm w"), _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"), pool.stride(0),
        _need(q_out, "q out", torch.bfloat16, (M, nh * hd)), M, nh, nkv, K, sp, n_sp, s_stride, dim, eps_norm,
        *(ahead or (None, 0)), _error_flag(x.device).data_ptr(), _stream()), "mv_gemm_tc_swap_heads")
    _account_gemm(x, w_qkv, q_out, False)
    return q_out


def shortconv(p: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
              positions, seq_of, cu, slots, starts, lens, out: torch.Tensor, n_seqs: int,
              decode: bool = False) -> torch.Tensor:
    """Gated short convolution between its projections; updates ``state``
    [n_slots, k-1, H] in place for the ``n_seqs`` sequences of the step.
    ``decode``: every sequence brings exactly one token (one fused kernel)."""
    N, H3 = p.shape
    H, k = w.shape
    if H3 != 3 * H:
        raise KernelError(f"shortconv: projection width {H3} is not 3 x {H}")
    if not 1 <= k <= MAX_CONV_K:
        raise KernelError(f"shortconv: convolution width {k} is outside 1..{MAX_CONV_K}")
    _need(state, "shortconv state", torch.float32)
    if state.dim() != 3 or state.shape[1] != k - 1 or state.shape[2] != H:
        raise KernelError(f"shortconv: state shape {tuple(state.shape)}, expected [slots, {k - 1}, {H}]")
    _guard("core", "shortconv", p.device, n_slots=state.shape[0])
    if N == n_seqs and decode:
        _check(_fn("core", "mv_shortconv_decode")(
            _need(p, "shortconv p", torch.float32), _need(w, "shortconv taps", torch.float32),
            _need(bias, "shortconv bias", torch.float32, (H,), True), state.data_ptr(),
            _need(slots, "slots", torch.int32), _need(out, "shortconv out", None, (N, H)), _dt(out), N, H, k,
            _stream()), "mv_shortconv_decode")
        account(_nbytes(p, out) + 2 * N * (k - 1) * H * 4)
        return out
    _check(_fn("core", "mv_shortconv")(
        _need(p, "shortconv p", torch.float32), _need(w, "shortconv taps", torch.float32),
        _need(bias, "shortconv bias", torch.float32, (H,), True), state.data_ptr(),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(cu, "cu", torch.int32), _need(slots, "slots", torch.int32),
        _need(starts, "starts", torch.int32), _need(lens, "lens", torch.int32),
        _need(out, "shortconv out", None, (N, H)), _dt(out), N, n_seqs, H, k, _stream()), "mv_shortconv")
    account(_nbytes(p, out) + 2 * n_seqs * (k - 1) * H * 4)
    return out


def _check_kv(pool: torch.Tensor, nkv: int, hd: int, page_size: int, what: str):
    if pool.dim() != 5 or tuple(pool.shape[1:]) != (2, nkv, page_size, hd):
        raise KernelError(f"{what}: cache pool shape {tuple(pool.shape)}, expected "
                          f"[pages, 2, {nkv}, {page_size}, {hd}]")
    if page_size & (page_size - 1):
        raise KernelError(f"{what}: page size {page_size} is not a power of two")


def qk_prepare(qkv: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
               inv_freq: Optional[torch.Tensor], half_split: bool, positions, seq_of, page_table,
               pool: torch.Tensor, q_out: torch.Tensor, nh: int, nkv: int, hd: int,
               append: bool = True) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotation, and the write of k and v into
    the paged cache; q comes out in the model's dtype."""
    N = qkv.shape[0]
    if hd % 2 or hd > MAX_HEAD_DIM:
        raise KernelError(f"qk_prepare: head size {hd} must be even and at most {MAX_HEAD_DIM}")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "qk_prepare")
    if pool.dtype != q_out.dtype:
        raise KernelError(f"qk_prepare: cache is {pool.dtype} but q is {q_out.dtype}")
    _need(page_table, "page table", torch.int32)
    _guard("core", "attention", qkv.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_qk_prepare")(
        _need(qkv, "qkv", torch.float32, (N, (nh + 2 * nkv) * hd)),
        _need(wq, "q norm weight", torch.float32, (hd,), True),
        _need(wk, "k norm weight", torch.float32, (hd,), True), float(eps),
        _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        page_table.data_ptr(), page_table.shape[1], page_size, _need(pool, "cache pool"),
        pool.stride(0), int(append), _need(q_out, "q out", None, (N, nh * hd)), _dt(q_out), N, nh, nkv, hd,
        _stream()), "mv_qk_prepare")
    account(_nbytes(qkv, q_out) + N * 2 * nkv * hd * pool.element_size())
    return q_out


def qk_prepare_q_only(qkv: torch.Tensor, wq: Optional[torch.Tensor], eps: float,
                      inv_freq: Optional[torch.Tensor], half_split: bool, positions, q_out: torch.Tensor,
                      nh: int, hd: int) -> torch.Tensor:
    """The same for a layer that has queries only (it reads another layer's cache)."""
    N = qkv.shape[0]
    if hd % 2 or hd > MAX_HEAD_DIM:
        raise KernelError(f"qk_prepare: head size {hd} must be even and at most {MAX_HEAD_DIM}")
    _check(_fn("core", "mv_qk_prepare")(
        _need(qkv, "q", torch.float32, (N, nh * hd)), _need(wq, "q norm weight", torch.float32, (hd,), True),
        None, float(eps), _need(inv_freq, "inv_freq", torch.float32, (hd // 2,), True), int(half_split),
        _need(positions, "positions", torch.int32), None, None, 0, 1, None, 0, 0,
        _need(q_out, "q out", None, (N, nh * hd)), _dt(q_out), N, nh, 0, hd, _stream()), "mv_qk_prepare")
    return q_out


def attention_generic(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of,
                      out: torch.Tensor, nh: int, nkv: int, hd: int, scale: float, window: int = 0):
    """Causal attention of every token of the step over its sequence's cache
    (which already holds the step's own keys), optional sliding window."""
    N = q.shape[0]
    if hd % 8 or hd > MAX_HEAD_DIM:
        raise KernelError(f"attention: head size {hd} must be a multiple of 8 and at most {MAX_HEAD_DIM}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _guard("core", "attention", q.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_attention_generic")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), _dt(q), N, nh, nkv, hd, float(scale), int(window),
        _stream()), "mv_attention_generic")
    return out


_n_sms = {}


def n_sms(device=None) -> int:
    """Multiprocessors of the device (asked once); 148 where no device can be asked (planning on a CPU)."""
    if device is None and _n_sms:
        if len(_n_sms) == 1:                      # the usual case, asked many times a step
            return next(iter(_n_sms.values()))
    if not torch.cuda.is_available():
        return 148
    key = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if key not in _n_sms:
        _n_sms[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _n_sms[key]


DECODE_ATTENTION_MAX_TOKENS = 128      # steps with more query tokens split the work over the queries,
DECODE_ATTENTION_MAX_QUERIES = 2       # unless no sequence brings more than this many (a large decode batch)


def attention_decode_plan(N: int, nh: int, nkv: int, context_cap: int = 0):
    """(query heads per block, head tiles per kv head, key splits) for a step of N
    query tokens.  Enough blocks to fill the GPU twice over; more when the cache
    can be long (``context_cap`` tokens, the reach of the step's page table), so
    that a warp has about eight runs of 32 keys.  The count depends on the page
    table's width, not on the lengths: a decode step's launches are recorded once
    per width and replayed as the cache grows."""
    G = nh // nkv
    gt = 1 if G <= 1 else (2 if G <= 2 else (4 if G <= 4 else 8))
    head_tiles = -(-G // gt)
    splits = -(-2 * n_sms() // max(1, N * nkv * head_tiles))
    splits = max(splits, -(-context_cap // (32 * 4 * 8)))
    return gt, head_tiles, max(1, min(32, splits))


def attention_decode(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of, out: torch.Tensor,
                     nh: int, nkv: int, hd: int, scale: float, window: int, ws, splits: Optional[int] = None):
    """The same contract as ``attention_generic``, for steps with few query
    tokens: work is split over the keys, and the heads of a group share the
    loads.  ``ws`` (a Workspace) supplies the scratch for the key splits."""
    N = q.shape[0]
    if hd % 8 or hd > MAX_HEAD_DIM:
        raise KernelError(f"attention: head size {hd} must be a multiple of 8 and at most {MAX_HEAD_DIM}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    gt, head_tiles, auto = attention_decode_plan(N, nh, nkv, page_table.shape[1] * page_size)
    splits = auto if splits is None else int(splits)
    part_o = ws.get("attn_part_o", (N * nh * splits * hd,), torch.float32)
    part_ml = ws.get("attn_part_ml", (N * nh * splits * 2,), torch.float32)
    tickets = ws.get_zeroed("attn_tickets", (N * nkv * head_tiles,), torch.int32)
    _guard("core", "attention_decode", q.device, n_pages=pool.shape[0])
    _check(_fn("core", "mv_attention_decode")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), _dt(q), part_o.data_ptr(), part_ml.data_ptr(),
        tickets.data_ptr(), N, nh, nkv, hd, float(scale), int(window), splits, gt, head_tiles, _stream()),
        "mv_attention_decode")
    return out


def attention_decode_tc_plan(N: int, nkv: int, context_cap: int) -> int:
    """Key splits for the tcgen05 decode attention: as many as it takes to give each of the
    GPU's multiprocessors its two blocks (more blocks than that only add set-up and merging:
    at 64 tokens of 520 cached ones, 29 us unsplit against 39 us in two), at least two key
    blocks of 128 a split.  Like ``attention_decode_plan`` it depends on the page table's
    reach, not on the lengths."""
    blocks = max(1, -(-context_cap // 128))
    want = (2 * n_sms()) // max(1, N * nkv)
    if blocks <= 8:
        return 1          # up to 1,024 cached tokens a split saves less than its merge kernel costs
    return max(1, min(64, want, blocks // 2))


DECODE_TC_MAX_GROUP = 16


def attention_decode_tc_supported(dtype: torch.dtype, hd: int, pool: torch.Tensor, window: int, nh: int,
                                  nkv: int) -> bool:
    """What the tcgen05 decode attention takes: as the tcgen05 prefill attention, and at most 16
    query heads a kv head (they are the 16 columns of its transposed scores)."""
    return (attention_prefill_tc_supported(dtype, hd, pool, window) and nkv > 0 and nh % nkv == 0
            and nh // nkv <= DECODE_TC_MAX_GROUP)


def attention_decode_tc(q: torch.Tensor, pool: torch.Tensor, page_table, positions, seq_of, out: torch.Tensor,
                        nh: int, nkv: int, hd: int, scale: float, ws, splits: Optional[int] = None):
    """Attention of single query tokens over long caches, both products on tcgen05 (bfloat16,
    head size 64, pages of 64 tokens, no window).  Same arguments and result as
    :func:`attention_decode`."""
    N = q.shape[0]
    if not attention_decode_tc_supported(q.dtype, hd, pool, 0, nh, nkv):
        raise KernelError(f"attention_decode_tc: needs bfloat16, head size 64, a dense pool of 64-token pages and "
                          f"at most 16 heads a kv head, got {q.dtype}, {hd}, pool {tuple(pool.shape)}, {nh}/{nkv}")
    _check_kv(pool, nkv, hd, 64, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    splits = attention_decode_tc_plan(N, nkv, page_table.shape[1] * 64) if splits is None else int(splits)
    part_o = ws.get("attn_part_o", (N * nh * splits * hd,), torch.float32)
    part_ml = ws.get("attn_part_ml", (N * nh * splits * 2,), torch.float32)
    _check(_fn("bf16", "mv_attention_decode_tc")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.shape[0] * 2 * nkv * 64,
        _need(page_table, "page table", torch.int32), page_table.shape[1],
        _need(positions, "positions", torch.int32), _need(seq_of, "seq_of", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), part_o.data_ptr(), part_ml.data_ptr(), N, nh, nkv,
        float(scale), splits, _error_flag(q.device).data_ptr(), _stream()), "mv_attention_decode_tc")
    if splits > 1:
        add_launches(1)                    # the kernel that merges the splits
    return out


PREFILL_ATTENTION_MAX_HEAD_DIM = 128


def attention_prefill_supported(dtype: torch.dtype, hd: int) -> bool:
    return dtype == torch.bfloat16 and hd % 16 == 0 and hd <= PREFILL_ATTENTION_MAX_HEAD_DIM


def attention_prefill(q: torch.Tensor, pool: torch.Tensor, page_table, cu, starts, out: torch.Tensor,
                      n_seqs: int, nh: int, nkv: int, hd: int, scale: float, window: int = 0):
    """Causal attention of a step with many query tokens on the tensor cores
    (bfloat16, head sizes 16..128 in steps of 16).  The step's tokens are packed
    sequence by sequence (``cu``), sequence b starting at position ``starts[b]``."""
    N = q.shape[0]
    if not attention_prefill_supported(q.dtype, hd):
        raise KernelError(f"attention_prefill: needs bfloat16 and a head size 16..128 in steps of 16, "
                          f"got {q.dtype}, {hd}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    page_size = pool.shape[3]
    _check_kv(pool, nkv, hd, page_size, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _guard("bf16", "attention_prefill", q.device, n_pages=pool.shape[0])
    _check(_fn("bf16", "mv_attention_prefill")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.stride(0),
        _need(page_table, "page table", torch.int32), page_table.shape[1], page_size,
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), N, n_seqs, nh, nkv, hd, float(scale), int(window),
        _stream()), "mv_attention_prefill")
    return out


def attention_prefill_tc_supported(dtype: torch.dtype, hd: int, pool: torch.Tensor, window: int) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 64, no window, and a
    dense cache pool [pages, 2, kv heads, 64, 64] that a 2-D tensor map can describe."""
    if DEBUG_CHECKS:
        return False            # a build with index checks runs the kernels that have them
    if dtype != torch.bfloat16 or hd != 64 or window != 0 or pool.dim() != 5 or pool.shape[3] != 64:
        return False
    rows = pool.shape[0] * 2 * pool.shape[2] * 64
    return pool.is_contiguous() and rows < 2 ** 31 and pool.data_ptr() % 16 == 0


def attention_prefill_tc(q: torch.Tensor, pool: torch.Tensor, page_table, cu, starts, out: torch.Tensor,
                         n_seqs: int, nh: int, nkv: int, hd: int, scale: float):
    """Causal attention of a step with many query tokens, both products on tcgen05
    (bfloat16, head size 64, pages of 64 tokens, no window).  Same arguments and
    result as :func:`attention_prefill`."""
    N = q.shape[0]
    if not attention_prefill_tc_supported(q.dtype, hd, pool, 0):
        raise KernelError(f"attention_prefill_tc: needs bfloat16, head size 64 and a dense pool of 64-token pages, "
                          f"got {q.dtype}, {hd}, pool {tuple(pool.shape)}")
    if nh % nkv:
        raise KernelError(f"attention: {nh} heads are not a multiple of {nkv} kv heads")
    _check_kv(pool, nkv, hd, 64, "attention")
    if q.dtype != pool.dtype or out.dtype != q.dtype:
        raise KernelError(f"attention: q {q.dtype}, cache {pool.dtype}, out {out.dtype} must agree")
    _check(_fn("bf16", "mv_attention_prefill_tc")(
        _need(q, "q", None, (N, nh * hd)), _need(pool, "cache pool"), pool.shape[0] * 2 * nkv * 64,
        _need(page_table, "page table", torch.int32), page_table.shape[1],
        _need(cu, "cu", torch.int32), _need(starts, "starts", torch.int32),
        _need(out, "attention out", None, (N, nh * hd)), N, n_seqs, nh, nkv, float(scale),
        _error_flag(q.device).data_ptr(), _stream()), "mv_attention_prefill_tc")
    return out


def sample_scratch_width(V: int) -> int:
    """Floats of scratch a row of V logits needs: V rounded up to the sampling block's 1,024 threads."""
    return -(-int(V) // 1024) * 1024


def sample(logits: torch.Tensor, work: torch.Tensor, out: torch.Tensor, *, temperature: float,
           top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
           presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
           recent: Optional[torch.Tensor] = None, n_recent: Optional[torch.Tensor] = None, seed: int = 0,
           streams: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None,
           ring: Optional[torch.Tensor] = None, ring_rows: Optional[torch.Tensor] = None,
           flag_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` [B, V] (float32, rows may be strided).  ``work``: scratch of
    ``sample_scratch_width(V)`` floats a row.  The recent tokens that the penalties look at come
    either from the caller (``recent`` [B, 64], ``n_recent``) or from ``ring`` [states, 128], which the
    kernel keeps itself: row b uses state ``ring_rows[b]``, looks at the places of its last
    min(steps[b], 64) steps and writes the token it samples to place steps[b] mod 128.
    ``flag_to`` (int32 [1] on the device): the kernel also copies the device's error flag there, so
    that it reaches the host with the tokens."""
    B, V = logits.shape
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 on a CUDA device with unit column stride")
    if work.dim() != 2 or work.shape[0] < B:
        raise KernelError(f"sample: scratch {tuple(work.shape)} has fewer rows than the {B} rows of logits")
    if ring is not None and (steps is None or recent is not None):
        raise KernelError("sample: a ring of recent tokens needs the rows' steps, and excludes a caller's recent tokens")
    if recent is not None and (recent.shape != (B, RECENT_MAX)):
        raise KernelError(f"sample: recent tokens shape {tuple(recent.shape)}, expected [{B}, {RECENT_MAX}]")
    _check(_fn("core", "mv_sample")(
        logits.data_ptr(), logits.stride(0),
        _need(work, "sample scratch", torch.float32, (None, sample_scratch_width(V))), B, V,
        float(temperature), int(top_k), float(top_p), float(min_p), float(repetition_penalty),
        float(presence_penalty), float(frequency_penalty),
        _need(recent, "recent", torch.int32, optional=True),
        _need(n_recent, "n_recent", torch.int32, (B,), True), int(seed) & ((1 << 64) - 1),
        _need(streams, "streams", torch.int32, (B,), True), _need(steps, "steps", torch.int32, (B,), True),
        _need(ring, "recent ring", torch.int32, (None, RECENT_RING), True),
        _need(ring_rows, "ring rows", torch.int32, (B,), ring is None),
        _need(out, "sample out", torch.int32, (B,)),
        _error_flag(logits.device).data_ptr() if flag_to is not None else None,
        _need(flag_to, "flag copy", torch.int32, (1,), True), _stream()), "mv_sample")
    account(B * V * 4)
    return out
