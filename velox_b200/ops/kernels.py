"""Python entry points of the hand-written CUDA kernels (ctypes over the C launchers).

Every function here takes torch tensors that already live on the GPU, checks what a wrong
call could silently get wrong (dtype, contiguity, sizes), and launches on the current torch
stream.  There is no fallback: without a CUDA device or without a working nvcc build these
functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build

_c_int = ctypes.c_int
_c_ll = ctypes.c_longlong
_c_f = ctypes.c_float
_ptr = ctypes.c_void_p

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_core = None
_attention = {}


class KernelError(RuntimeError):
    pass


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "velox_b200 runs on a CUDA device only (sm_100a); no CUDA device is available "
            "and there is no CPU path"
        )


def core():
    global _core
    if _core is None:
        lib = build.load_core()
        lib.vx_embed.argtypes = [_ptr, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr]
        lib.vx_add_rmsnorm.argtypes = [
            _ptr, _ptr, _ptr, _c_f, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr,
        ]
        lib.vx_rope_cache_write.argtypes = [
            _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_swiglu.argtypes = [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr]
        lib.vx_gemm_f32.argtypes = [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr]
        lib.vx_cast_bf16_to_f32.argtypes = [_ptr, _ptr, _c_ll, _ptr]
        lib.vx_sample.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr,
            _ptr,
        ]
        lib.vx_sample_segments.argtypes = [_c_int, _c_int]
        lib.vx_selftest_bounded_wait.argtypes = [_ptr, _c_ll, _ptr, _ptr]
        lib.vx_gemm_bf16_add_mirrored.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_mlp_fused.argtypes = [
            _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_ll, _c_int, _c_int, _c_int, _ptr, _ptr,
        ]
        lib.vx_filter_threshold.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr,
        ]
        lib.vx_apply_penalties.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_glu.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_f, _c_f, _c_f, _c_f, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_xielu.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_int, _c_f, _c_f, _c_int,
            _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_add_chunked.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_normed.argtypes = [
            _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_norm_rows.argtypes = [_ptr, _ptr, _ptr, _c_f, _c_int, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr]
        lib.vx_gated_norm_add.argtypes = [
            _ptr, _ptr, _ptr, _c_ll, _ptr, _c_ll, _ptr, _c_f, _c_int, _ptr, _c_int, _ptr, _c_ll, _ptr, _c_int, _ptr,
            _c_int, _c_int, _ptr, _c_ll, _ptr, _ptr,
        ]
        lib.vx_xielu.argtypes = [_ptr, _c_ll, _ptr, _c_int, _c_int, _c_int, _c_f, _c_f, _ptr]
        lib.vx_softcap.argtypes = [_ptr, _c_ll, _c_f, _ptr]
        lib.vx_cast_f32_to_bf16.argtypes = [_ptr, _ptr, _c_ll, _ptr]
        lib.vx_rms_rows.argtypes = [_ptr, _c_ll, _c_int, _ptr, _c_f, _c_int, _ptr, _c_ll, _c_int, _c_int, _ptr]
        lib.vx_latent_prepare.argtypes = [
            _ptr, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _ptr, _c_f, _ptr, _ptr, _c_ll,
            _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr,
        ]
        lib.vx_headwise_linear.argtypes = [
            _ptr, _c_ll, _c_int, _ptr, _ptr, _c_ll, _c_int, _ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
            _ptr,
        ]
        lib.vx_gemm_bf16_qkv_rope.argtypes = [
            _ptr, _c_int, _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _c_int,
            _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _c_ll, _c_int, _c_int, _ptr, _ptr,
        ]
        _core = lib
    return _core


_mixers = None


def mixers():
    """The library of recurrent mixers and expert feed-forwards (built at first use)."""
    global _mixers
    if _mixers is None:
        lib = build.load_mixers()
        lib.vx_pair_rope_cache_write.argtypes = [
            _ptr, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
            _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_head_gate.argtypes = [_ptr, _c_int, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_int, _ptr]
        lib.vx_conv_tokens.argtypes = [
            _ptr, _c_int, _c_ll, _c_int, _c_int, _ptr, _ptr, _ptr, _c_ll, _ptr, _c_ll, _ptr, _ptr, _ptr, _c_int,
            _c_int, _c_int, _ptr,
        ]
        lib.vx_rglru_gates.argtypes = [
            _ptr, _c_ll, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_f, _ptr, _ptr, _c_ll, _c_int, _ptr, _ptr,
            _ptr,
        ]
        lib.vx_rglru_scan.argtypes = [
            _ptr, _ptr, _c_ll, _ptr, _c_int, _c_ll, _c_int, _ptr, _c_ll, _ptr, _c_ll, _ptr, _ptr, _ptr, _c_int,
            _c_int, _ptr, _c_int, _ptr,
        ]
        lib.vx_rglru_chunk_rows.restype = _c_int
        lib.vx_ssd_scan.argtypes = [
            _ptr, _c_ll, _ptr, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_int,
            _c_int, _ptr, _ptr, _ptr, _c_int, _ptr, _c_int, _ptr,
        ]
        lib.vx_ssd_chunk_rows.restype = _c_int
        lib.vx_gated_group_norm.argtypes = [
            _ptr, _c_ll, _ptr, _c_int, _c_ll, _ptr, _c_f, _c_int, _c_int, _ptr, _c_ll, _c_int, _c_int, _ptr,
        ]
        lib.vx_delta_rule_scan.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_ll, _ptr, _c_ll, _ptr, _ptr, _c_f, _c_f, _ptr, _c_ll, _ptr, _c_ll, _ptr,
            _c_ll, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _ptr, _c_ll, _ptr, _ptr,
        ]
        lib.vx_delta_rule_chunk_scratch.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int]
        lib.vx_delta_rule_chunk_scratch.restype = _c_ll
        lib.vx_delta_rule_packed_width.argtypes = [_c_int, _c_int, _c_int]
        lib.vx_delta_rule_packed_width.restype = _c_int
        lib.vx_dual_norm_mean.argtypes = [_ptr, _ptr, _c_int, _ptr, _ptr, _c_f, _c_f, _c_int, _ptr, _ptr, _c_int, _ptr]
        lib.vx_act_rows.argtypes = [_ptr, _c_int, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_int, _ptr]
        lib.vx_residual_add.argtypes = [_ptr, _ptr, _c_int, _c_ll, _ptr]
        lib.vx_gated_rows_add.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_ll, _c_int, _c_int, _ptr]
        lib.vx_table_experts.argtypes = [
            _ptr, _c_int, _c_ll, _ptr, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _ptr,
            _c_int, _ptr, _ptr,
        ]
        lib.vx_table_experts_rows.argtypes = [
            _ptr, _c_int, _c_ll, _ptr, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _ptr,
            _ptr, _c_int, _ptr, _ptr,
        ]
        lib.vx_grouped_tile_rows.restype = _c_int
        lib.vx_table_experts_grouped.argtypes = [
            _ptr, _c_ll, _ptr, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _ptr, _c_int,
            _ptr, _c_ll, _ptr, _ptr, _c_int, _ptr, _ptr,
        ]
        lib.vx_route_and_gather.argtypes = [
            _ptr, _c_ll, _ptr, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _c_int,
            _ptr, _ptr,
        ]
        lib.vx_gather_pairs.argtypes = [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _c_int, _ptr]
        _mixers = lib
    return _mixers


_heads = None


def heads():
    """The library of row kernels around attention heads and gated feed-forwards (built at first use)."""
    global _heads
    if _heads is None:
        lib = build.load_heads()
        lib.vx_norm_shift.argtypes = [
            _ptr, _c_ll, _c_int, _c_f, _ptr, _ptr, _ptr, _ptr, _c_ll, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _c_int,
            _c_int, _ptr,
        ]
        lib.vx_add_rows.argtypes = [_ptr, _ptr, _ptr, _c_int, _c_ll, _c_f, _c_f, _ptr]
        lib.vx_norm_conv.argtypes = [
            _ptr, _c_ll, _c_int, _c_f, _ptr, _ptr, _c_int, _ptr, _c_ll, _ptr, _c_int, _ptr, _ptr, _ptr, _c_int,
            _c_int, _ptr,
        ]
        lib.vx_diff_prepare.argtypes = [
            _ptr, _c_int, _c_ll, _ptr, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _c_f, _ptr, _ptr, _ptr, _c_int, _c_int,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_diff_combine.argtypes = [
            _ptr, _c_int, _c_ll, _ptr, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_f, _c_f, _c_f, _ptr,
        ]
        lib.vx_clamped_glu.argtypes = [_ptr, _c_int, _c_ll, _ptr, _c_ll, _c_int, _c_int, _c_f, _c_f, _c_f, _c_f, _ptr]
        _heads = lib
    return _heads


def attention_lib(head_dim: int):
    lib = _attention.get(head_dim)
    if lib is None:
        lib = build.load_attention(head_dim)
        lib.vx_attention_scored.argtypes = [
            _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_f, _c_int, _c_int, _c_f, _ptr, _ptr,
            _c_int, _c_int, _ptr, _c_int, _ptr,
        ]
        lib.vx_attention.argtypes = [
            _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_f, _c_int, _c_int, _ptr,
        ]
        lib.vx_attn_has_tc.restype = _c_int
        lib.vx_attn_narrow_ctas_per_sm.restype = _c_int
        lib.vx_attn_max_cluster.restype = _c_int
        lib.vx_attn_narrow_max_active_clusters.restype = _c_int
        lib.vx_attn_narrow_max_active_clusters.argtypes = [_c_int]
        lib.vx_attention_merge.argtypes = [
            _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr,
        ]
        lib.vx_attn_head_dim.restype = _c_int
        if lib.vx_attn_head_dim() != head_dim:
            raise KernelError(f"attention library for head size {head_dim} reports another size")
        _attention[head_dim] = lib
    return lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current device's current stream (asked for at every launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# Launcher calls made so far (each is at least one kernel of this package).
launch_count = 0

# While this is a list, every launcher call appends (launcher name, a CUDA event recorded right
# after its launch).  With the host running ahead of the device (the caller queues a delay
# first), the time between consecutive events is the device time of each launch, without a
# profiler.  An event between two kernels also keeps the second from starting early, so the
# times are those of kernels that run one after the other.
launch_events: Optional[list] = None


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    if launch_events is not None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        launch_events.append((what, event))


def note_library_launch(what: str) -> None:
    """Called after a library kernel (a cuBLAS product through torch) has been queued, so that a
    timeline of ``launch_events`` has an entry for it too.  It does not count as a launch of
    this package's kernels."""
    if launch_events is not None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        launch_events.append((what, event))


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype is dtype and t.is_cuda and t.is_contiguous():
        return
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"compute dtype must be float32 or bfloat16, got {dtype}") from None


# ------------------------------------------------------------------------------------------
def selftest_bounded_wait(status: torch.Tensor, limit_cycles: int) -> int:
    """Run one CTA that waits, with a limit of ``limit_cycles`` SM cycles, on a barrier nobody
    arrives at.  Returns 1 when the wait gave up (and set its bit in ``status``), 2 if the
    barrier flipped, 0 if the kernel never reported.  Synchronises."""
    _need(status, torch.int32, "status")
    returned = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(core().vx_selftest_bounded_wait(_p(status), int(limit_cycles), _p(returned), _stream()),
           "selftest_bounded_wait")
    return int(returned.item())


def embed(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, status: torch.Tensor,
          fed: Optional[torch.Tensor] = None) -> None:
    """resid[t, :] = float32(table[ids[t], :]); ids outside the table set a status bit.

    With ``fed`` (int32 on the device: the tokens the sampler drew in the step before, one per
    row) an id of ``-1 - r`` stands for ``fed[r]`` and is looked up on the device."""
    _need(ids, torch.int32, "ids")
    if fed is not None:
        _need(fed, torch.int32, "fed")
    _need(resid, torch.float32, "resid")
    _need(table, table.dtype, "table")
    vocab, hidden = table.shape
    n = ids.numel()
    if resid.shape[0] < n or resid.shape[1] != hidden:
        raise ValueError(f"resid {tuple(resid.shape)} cannot hold {n} rows of width {hidden}")
    _check(
        core().vx_embed(_p(table), _code(table.dtype), _p(ids), _p(resid), n, hidden, vocab,
                        _p(status), _p(fed), 0 if fed is None else fed.numel(), _stream()),
        "embed",
    )


def add_rmsnorm(
    resid: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    num_rows: int,
    rows: Optional[torch.Tensor] = None,
    write_resid: bool = True,
) -> None:
    """v = resid + delta; resid = v (if write_resid); out = rmsnorm(v) * weight, float32 inside.

    ``delta`` is a pending product in the compute dtype, or None.  With ``rows`` (int32
    indices), output row o is computed from input row rows[o].
    """
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(out, out.dtype, "out")
    hidden = resid.shape[1]
    if weight.numel() != hidden or out.shape[1] != hidden:
        raise ValueError("norm weight / output width does not match the residual width")
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[1] != hidden:
            raise ValueError("delta width does not match the residual width")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < num_rows:
            raise ValueError(f"{num_rows} rows asked for, the index array names {rows.numel()}")
    elif resid.shape[0] < num_rows or (delta is not None and delta.shape[0] < num_rows):
        raise ValueError(f"{num_rows} rows asked for, the input has {resid.shape[0]}")
    if out.shape[0] < num_rows:
        raise ValueError(f"{num_rows} rows asked for, the output holds {out.shape[0]}")
    _check(
        core().vx_add_rmsnorm(_p(resid), _p(delta), _p(weight), float(eps), _p(out),
                              _code(out.dtype), _p(rows), num_rows, hidden,
                              1 if write_resid else 0, _stream()),
        "add_rmsnorm",
    )


def norm_rows(
    resid: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    center: bool,
    out: torch.Tensor,
    num_rows: int,
    rows: Optional[torch.Tensor] = None,
    write_resid: bool = True,
) -> None:
    """v = resid + delta; resid = v (if write_resid); out = norm(v) * weight in float32, where
    norm takes the mean off first when ``center`` is set (layer norm without bias) and divides
    by sqrt(mean of squared deviations + eps).  ``rows`` as in ``add_rmsnorm``."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(out, out.dtype, "out")
    hidden = resid.shape[1]
    if weight.numel() != hidden or out.shape[1] != hidden:
        raise ValueError("norm weight / output width does not match the residual width")
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[1] != hidden:
            raise ValueError("delta width does not match the residual width")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < num_rows:
            raise ValueError(f"{num_rows} rows asked for, the index array names {rows.numel()}")
    elif resid.shape[0] < num_rows or (delta is not None and delta.shape[0] < num_rows):
        raise ValueError(f"{num_rows} rows asked for, the input has {resid.shape[0]}")
    if out.shape[0] < num_rows:
        raise ValueError(f"{num_rows} rows asked for, the output holds {out.shape[0]}")
    _check(
        core().vx_norm_rows(_p(resid), _p(delta), _p(weight), float(eps), 1 if center else 0, _p(out),
                            _code(out.dtype), _p(rows), num_rows, hidden, 1 if write_resid else 0, _stream()),
        "norm_rows",
    )


def _rows_view(t: torch.Tensor, name: str, dtype: torch.dtype, num_rows: int, width: int) -> int:
    """Checks a [rows, >= width] view with unit column stride; returns its row pitch."""
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] < width or t.shape[0] < num_rows:
        raise ValueError(f"{name} must be device rows [>= {num_rows}, >= {width}] with unit column stride, "
                         f"got {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def gated_norm_add(
    resid_in: torch.Tensor,
    resid_out: torch.Tensor,
    delta: torch.Tensor,
    gate: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    center: bool,
    num_rows: int,
    lowp_out: Optional[torch.Tensor] = None,
    history: Optional[torch.Tensor] = None,
    mix_weights: Optional[torch.Tensor] = None,
    mix_out: Optional[torch.Tensor] = None,
    sums: Optional[torch.Tensor] = None,
    sums_bias: Optional[torch.Tensor] = None,
    compute_dtype: Optional[torch.dtype] = None,
) -> None:
    """A sublayer's result joins the float32 stream: ``y = delta * sigmoid(gate)`` (``gate``
    None: ``y = delta``), ``resid_out = resid_in + norm(y) * weight``.  ``delta`` and ``gate``
    are rows in the compute dtype and may be column ranges of wider buffers.

    Instead of ``delta`` the result may lie in ``sums``, float32 rows into which a projection has
    added its shares (``delta`` None, ``compute_dtype`` given): then ``y`` is made from ``sums +
    sums_bias`` and the rows read are set to zero again.

    With ``mix_weights`` (float32 [n]) what goes on is ``sum_{j < n-1} mix_weights[j] *
    history[j] + mix_weights[n-1] * resid_out`` (``history`` float32 [>= n-1, rows, width]: the
    kept results of earlier layers), written to ``mix_out``.  ``lowp_out`` gets what goes on
    (the mixed rows, or ``resid_out`` without a mix) in the compute dtype."""
    _need(resid_in, torch.float32, "resid_in")
    _need(resid_out, torch.float32, "resid_out")
    _need(weight, torch.float32, "weight")
    hidden = resid_in.shape[1]
    if resid_out.shape[1] != hidden or weight.numel() != hidden:
        raise ValueError("gated_norm_add: widths do not agree")
    if resid_in.shape[0] < num_rows or resid_out.shape[0] < num_rows:
        raise ValueError(f"gated_norm_add: {num_rows} rows asked for")
    if (delta is None) == (sums is None):
        raise ValueError("gated_norm_add takes the result either as delta or as float32 sums")
    sums_ld = 0
    if sums is not None:
        if compute_dtype is None:
            raise ValueError("gated_norm_add: float32 sums need the compute dtype named")
        dtype = compute_dtype
        sums_ld = _rows_view(sums, "sums", torch.float32, num_rows, hidden)
        delta_ld = 0
        if sums_bias is not None:
            _need(sums_bias, torch.float32, "sums_bias")
            if sums_bias.numel() != hidden:
                raise ValueError("gated_norm_add: the bias has another width than the rows")
    else:
        dtype = delta.dtype
        delta_ld = _rows_view(delta, "delta", dtype, num_rows, hidden)
    gate_ld = 0 if gate is None else _rows_view(gate, "gate", dtype, num_rows, hidden)
    if lowp_out is not None:
        _need(lowp_out, dtype, "lowp_out")
        if lowp_out.shape[1] != hidden or lowp_out.shape[0] < num_rows:
            raise ValueError("gated_norm_add: lowp_out does not hold the rows")
    terms, hist_stride = 0, 0
    if mix_weights is not None:
        _need(mix_weights, torch.float32, "mix_weights")
        terms = mix_weights.numel()
        if mix_out is None:
            raise ValueError("gated_norm_add: a mix needs mix_out")
        _need(mix_out, torch.float32, "mix_out")
        if mix_out.shape[1] != hidden or mix_out.shape[0] < num_rows:
            raise ValueError("gated_norm_add: mix_out does not hold the rows")
        if terms > 1:
            _need(history, torch.float32, "history")
            if history.dim() != 3 or history.shape[0] < terms - 1 or history.shape[1] < num_rows or history.shape[2] != hidden:
                raise ValueError(f"gated_norm_add: history {tuple(history.shape)} does not hold {terms - 1} results")
            hist_stride = history.stride(0)
    _check(
        core().vx_gated_norm_add(_p(resid_in), _p(resid_out), _p(delta), delta_ld, _p(gate), gate_ld, _p(weight),
                                 float(eps), 1 if center else 0, _p(lowp_out), _code(dtype), _p(history), hist_stride,
                                 _p(mix_weights), terms, _p(mix_out), num_rows, hidden, _p(sums), sums_ld,
                                 _p(sums_bias) if sums is not None else None, _stream()),
        "gated_norm_add",
    )


def xielu(x: torch.Tensor, out: torch.Tensor, num_rows: int, a_pos: float, a_neg: float) -> None:
    """out[t, i] = a_pos z^2 + z / 2 for z = x[t, i] > 0, else a_neg (exp(z) - 1 - z) + z / 2;
    ``x`` may be a column range of a wider buffer, ``out`` is dense [rows, n]."""
    _need(out, out.dtype, "out")
    n = out.shape[1]
    ld = _rows_view(x, "x", out.dtype, num_rows, n)
    if out.shape[0] < num_rows:
        raise ValueError("xielu: out does not hold the rows")
    _check(core().vx_xielu(_p(x), ld, _p(out), _code(out.dtype), num_rows, n, float(a_pos), float(a_neg), _stream()),
           "xielu")


def softcap(values: torch.Tensor, num_rows: int, cap: float) -> None:
    """values[:num_rows] = cap * tanh(values / cap), in place (float32)."""
    _need(values, torch.float32, "values")
    _check(core().vx_softcap(_p(values), num_rows * values.shape[1], float(cap), _stream()), "softcap")


def cast_f32_to_bf16(src: torch.Tensor, out: torch.Tensor, count: int) -> None:
    _need(src, torch.float32, "src")
    _need(out, torch.bfloat16, "out")
    _check(core().vx_cast_f32_to_bf16(_p(src), _p(out), count, _stream()), "cast")


def latent_prepare(
    proj: torch.Tensor,
    q_offset: int,
    latent_offset: Optional[int],
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    latent_weight: Optional[torch.Tensor],
    eps: float,
    slots: Optional[torch.Tensor],
    cache: Optional[torch.Tensor],
    queries: torch.Tensor,
    num_tokens: int,
    num_heads: int,
    dim: int,
    rot_dim: int,
    kv_rank: int,
    status: torch.Tensor,
    half_layout: bool = False,
    q_source: Optional[torch.Tensor] = None,
) -> None:
    """What a latent-attention layer does to its projections before attention (latent.cu).

    ``proj`` [T, width]: head h's query at ``q_offset + h * (dim + rot_dim)``, its last
    ``rot_dim`` dims rotate; the token's latent (``kv_rank`` values) and shared key part
    (``rot_dim`` values) at ``latent_offset`` (None: the layer reads another layer's cache).
    ``queries`` [T, heads, D]: dims ``kv_rank ...`` get the rotated parts and zero padding.
    ``cache`` [pages, page, 1, D]: the token's row at ``slots[t]`` gets [rms-normed latent |
    rotated key part | zeros]; a negative slot writes nothing.  ``half_layout``: dim i of a rotated
    part is paired with dim i + pairs, not dims 2i and 2i + 1.  ``q_source`` [T, width']: the
    queries come from this buffer (a projection of their own) at ``q_offset``, not from ``proj``."""
    dtype = proj.dtype
    _need(proj, dtype, "proj")
    _need(queries, dtype, "queries")
    _need(positions, torch.int32, "positions")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    if q_source is not None:
        _need(q_source, dtype, "q_source")
    padded = queries.shape[-1]
    if queries.numel() < num_tokens * num_heads * padded or proj.shape[0] < num_tokens:
        raise ValueError("latent_prepare: buffers do not hold the tokens")
    write = latent_offset is not None
    num_slots = 0
    if write:
        _need(cache, dtype, "cache")
        _need(slots, torch.int32, "slots")
        _need(latent_weight, torch.float32, "latent_weight")
        if cache.shape[-1] != padded or cache.shape[2] != 1 or latent_weight.numel() != kv_rank:
            raise ValueError("latent_prepare: cache rows or norm weight do not match the sizes")
        num_slots = cache.shape[0] * cache.shape[1]
    _check(
        core().vx_latent_prepare(_p(proj), proj.stride(0), _p(q_source),
                                 0 if q_source is None else q_source.stride(0), int(q_offset), int(latent_offset) if write else -1,
                                 _code(dtype), _p(positions), _p(cos), _p(sin), cos.shape[0], cos.shape[1],
                                 _p(latent_weight) if write else None, float(eps), _p(slots) if write else None,
                                 _p(cache) if write else None, num_slots, _p(queries), num_tokens, num_heads, dim,
                                 rot_dim, kv_rank, padded, 1 if half_layout else 0, _p(status), _stream()),
        "latent_prepare",
    )


def rms_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, num_tokens: int) -> None:
    """out[t, i] = x[t, i] / sqrt(mean(x[t]^2) + eps) * weight[i]; ``x`` may be a column range of a wider
    buffer; columns of ``out`` beyond the width of ``x`` are set to zero."""
    _need(weight, torch.float32, "weight")
    n = x.shape[1]
    if weight.numel() != n or out.dtype != x.dtype or out.shape[1] < n:
        raise ValueError("rms_rows: widths do not agree")
    _check(core().vx_rms_rows(_p(x), _pitched(x, "x"), _code(x.dtype), _p(weight), float(eps), n, _p(out),
                              _pitched(out, "out"), out.shape[1], num_tokens, _stream()), "rms_rows")


def headwise_linear(
    x: torch.Tensor,
    x_offset: int,
    x_head_stride: int,
    weight: torch.Tensor,
    out: torch.Tensor,
    out_offset: int,
    out_head_stride: int,
    num_tokens: int,
    gate: Optional[torch.Tensor] = None,
    gate_offset: int = 0,
    gate_each: bool = False,
) -> None:
    """out[t, out_offset + h * out_head_stride + n] = sum_k weight[h, n, k] * x[t, x_offset + h *
    x_head_stride + k], times sigmoid(gate[t, gate_offset + h]) with a gate, or, with ``gate_each``,
    times sigmoid(gate[t, gate_offset + h * N + n]): a logit per output.  ``x``, ``out`` and
    ``gate`` are dense 2-D buffers in the dtype of ``weight`` [heads, N, K]; float32 sums."""
    dtype = weight.dtype
    _need(weight, dtype, "weight")
    _need(x, dtype, "x")
    _need(out, dtype, "out")
    heads, n, k = weight.shape
    if x_offset + (heads - 1) * x_head_stride + k > x.shape[1] or out_offset + (heads - 1) * out_head_stride + n > out.shape[1]:
        raise ValueError("headwise_linear: the heads do not fit the rows")
    if x.shape[0] < num_tokens or out.shape[0] < num_tokens:
        raise ValueError("headwise_linear: buffers do not hold the tokens")
    gate_ptr, gate_ld = None, 0
    if gate is not None:
        _need(gate, dtype, "gate")
        if gate_offset + heads * (n if gate_each else 1) > gate.shape[1]:
            raise ValueError("headwise_linear: the gate columns do not fit the rows")
        gate_ptr, gate_ld = gate.data_ptr() + gate_offset * gate.element_size(), gate.stride(0)
    code = core().vx_headwise_linear(x.data_ptr() + x_offset * x.element_size(), x.stride(0), x_head_stride,
                                     _p(weight), out.data_ptr() + out_offset * out.element_size(), out.stride(0),
                                     out_head_stride, gate_ptr, gate_ld, _code(dtype), num_tokens, heads, n, k,
                                     1 if gate_each else 0, _stream())
    if code == -1:
        raise KernelError(f"headwise_linear refuses an inner size of {k}")
    _check(code, "headwise_linear")


def rope_cache_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_tokens: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    status: torch.Tensor,
    values_from_keys: bool = False,
) -> None:
    """Rotate q in place; rotate k and write k, v to the paged cache at ``slots``.

    ``k_cache``/``v_cache`` None: rotate q only (a layer that reads another layer's cache).
    ``values_from_keys``: the rows hold q | k only; a token's values are its keys as they stand in
    the row (k is rotated on its way into the cache, never in the row).
    """
    _need(qkv, qkv.dtype, "qkv")
    _need(positions, torch.int32, "positions")
    _need(slots, torch.int32, "slots")
    if qkv.shape[1] != (num_heads + (1 if values_from_keys else 2) * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not match the head counts")
    write = k_cache is not None
    if write:
        _need(k_cache, qkv.dtype, "k_cache")
        _need(v_cache, qkv.dtype, "v_cache")
        num_slots = k_cache.shape[0] * k_cache.shape[1]
    else:
        num_slots = 0
    if rotary_dim > 0:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        max_pos = cos.shape[0]
        if cos.shape[1] != rotary_dim // 2:
            raise ValueError("cos/sin tables do not match the rotary width")
    else:
        max_pos = 0
    _check(
        core().vx_rope_cache_write(_p(qkv), _code(qkv.dtype), _p(positions), _p(cos), _p(sin),
                                   _p(slots), _p(k_cache), _p(v_cache), num_tokens, num_heads,
                                   num_kv_heads, head_dim, rotary_dim, max_pos, num_slots,
                                   1 if write else 0, qkv.stride(0), 1 if values_from_keys else 0, _p(status),
                                   _stream()),
        "rope_cache_write",
    )


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, num_tokens: int) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need(gate_up, gate_up.dtype, "gate_up")
    _need(out, gate_up.dtype, "out")
    inter = out.shape[1]
    if gate_up.shape[1] != 2 * inter:
        raise ValueError("gate_up must be twice as wide as the output")
    _check(
        core().vx_swiglu(_p(gate_up), _p(out), _code(out.dtype), num_tokens, inter, _stream()),
        "swiglu",
    )


def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
             num_rows: int) -> None:
    """out[:M] = a[:M] @ w.T + bias on the FP32 pipes (true 32-bit, no tensor cores)."""
    _need(a, torch.float32, "a")
    _need(w, torch.float32, "w")
    _need(out, torch.float32, "out")
    n, k = w.shape
    if a.shape[1] != k or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != n:
            raise ValueError("bias length does not match the output width")
    _check(core().vx_gemm_f32(_p(a), _p(w), _p(bias), _p(out), num_rows, n, k, _stream()), "gemm_f32")


GEMM_OUT_BF16, GEMM_OUT_F32, GEMM_ADD_F32, GEMM_SWIGLU = 0, 1, 2, 3


def gemm_bf16_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel moves tiles with TMA: rows must be 16-byte multiples."""
    return w.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_bf16(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    mode: int,
    num_rows: int,
    status: torch.Tensor,
    splits: int = 1,
) -> None:
    """out = x[:num_rows] @ w.T on tcgen05 tensor cores (see gemm_bf16.cu for the modes).

    ``splits`` CTAs (1, 2, 4 or 8; rounded down) share each output tile as a thread-block
    cluster and reduce through distributed shared memory; the output is final either way.
    """
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    n, k = w.shape
    if mode == GEMM_SWIGLU:
        if n % 2:
            raise ValueError("a gate/up matrix needs an even number of rows")
        n //= 2
    if x.shape[1] != k:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    want = torch.bfloat16 if mode in (GEMM_OUT_BF16, GEMM_SWIGLU) else torch.float32
    _need(out, want, "out")
    if out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"output {tuple(out.shape)} does not match width {n}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    code = core().vx_gemm_bf16(_p(x), _p(w), _p(bias), _p(out), mode, num_rows, x.shape[0], n, k,
                               out.stride(0), splits, _p(status), _stream())
    if code == -1:
        raise KernelError(
            f"gemm_bf16 refuses x {tuple(x.shape)} w {tuple(w.shape)}: the inner size must be a "
            "multiple of 8 and both operands 16-byte aligned"
        )
    _check(code, "gemm_bf16")


def gemm_bf16_glu(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, num_rows: int,
                  limit: float, alpha: float, up_shift: float, status: torch.Tensor, cubic: float = 0.0) -> None:
    """out[:num_rows] = g * sigmoid(alpha * (g + cubic * g^3)) * (u + up_shift) with g and u the two halves of
    x[:num_rows] @ w.T + bias (w [2 F, K]: the F gate rows, then the F up rows; bias [2 F] float32
    or None), g cut at ``limit`` from above and u to +-``limit`` when ``limit`` > 0, in the
    epilogue of the tcgen05 kernel: the activations' inputs never leave the SM."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16, "out")
    n, k = w.shape
    if n % 2 or x.shape[1] != k or out.dim() != 2 or out.shape[1] != n // 2:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != n:
            raise ValueError(f"bias of {bias.numel()} elements for {n} rows")
    code = core().vx_gemm_bf16_glu(_p(x), _p(w), _p(bias), _p(out), num_rows, x.shape[0], n // 2, k, out.stride(0),
                                   float(limit), float(alpha), float(up_shift), float(cubic), _p(status), _stream())
    if code == -1:
        raise KernelError(f"gemm_bf16_glu refuses x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(code, "gemm_bf16_glu")


def gemm_bf16_xielu(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    act_out: torch.Tensor,
    act_from: int,
    a_pos: float,
    a_neg: float,
    num_rows: int,
    status: torch.Tensor,
    splits: int = 1,
) -> bool:
    """``x[:num_rows] @ w.T + bias`` on the tensor-core kernel with the xIELU activation in its
    epilogue: columns below ``act_from`` go to ``out`` as they are, the others, activated, to the
    dense ``act_out`` [rows, N - act_from].  False (nothing launched) for sizes the kernel refuses."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16, "out")
    _need(act_out, torch.bfloat16, "act_out")
    n, k = w.shape
    if x.shape[1] != k or out.shape[1] < act_from or act_out.shape[1] != n - act_from:
        raise ValueError(f"gemm_bf16_xielu shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, "
                         f"out {tuple(out.shape)}, act_out {tuple(act_out.shape)}, act_from {act_from}")
    if out.shape[0] < num_rows or act_out.shape[0] < num_rows:
        raise ValueError("gemm_bf16_xielu: outputs do not hold the rows")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    code = core().vx_gemm_bf16_xielu(_p(x), _p(w), _p(bias), _p(out), _p(act_out), num_rows, x.shape[0], n, k,
                                     out.stride(0), act_out.stride(0), int(act_from), float(a_pos), float(a_neg),
                                     int(splits), _p(status), _stream())
    if code == -1:
        return False
    _check(code, "gemm_bf16_xielu")
    return True


def gemm_bf16_add_chunked(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, num_rows: int,
                          status: torch.Tensor, chunks: int, bias: Optional[torch.Tensor] = None) -> None:
    """out[:num_rows] += x[:num_rows] @ w.T (+ bias) (float32 ``out``) with the inner dimension cut into
    ``chunks`` ranges taken by independent CTAs, which add their partial tiles to ``out`` by
    reductions at the L2: any number of CTAs per output tile, no cluster, and an order of
    additions that is not fixed."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.float32, "out")
    n, k = w.shape
    if x.shape[1] != k or out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != n:
            raise ValueError(f"bias of {bias.numel()} elements for {n} outputs")
    code = core().vx_gemm_bf16_add_chunked(_p(x), _p(w), _p(bias), _p(out), num_rows, x.shape[0], n, k, out.stride(0),
                                           int(chunks), _p(status), _stream())
    if code == -1:
        raise KernelError(f"gemm_bf16_add_chunked refuses x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(code, "gemm_bf16_add_chunked")


# Steps of at most this many tokens can have their input norm made inside the projection.
GEMM_NORMED_MAX_TOKENS = 64


def gemm_bf16_normed(
    resid: torch.Tensor,
    norm_weight: torch.Tensor,
    eps: float,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    mode: int,
    num_rows: int,
    status: torch.Tensor,
    splits: int = 1,
) -> bool:
    """``gemm_bf16`` on ``rmsnorm(resid[:num_rows]) * norm_weight`` without that tensor ever
    existing: the kernel makes the bf16 tiles from the float32 rows and applies 1 / rms to its
    accumulator.  At most ``GEMM_NORMED_MAX_TOKENS`` rows.  False (and nothing launched) when
    the tiles of a row this long do not fit in shared memory."""
    if resid.dtype != torch.float32 or resid.dim() != 2 or resid.stride(1) != 1:
        raise TypeError("resid must be float32 rows")
    _need(norm_weight, torch.float32, "norm_weight")
    _need(w, torch.bfloat16, "w")
    n, k = w.shape
    if mode == GEMM_SWIGLU:
        if n % 2:
            raise ValueError("a gate/up matrix needs an even number of rows")
        n //= 2
    if resid.dim() != 2 or resid.shape[1] != k or norm_weight.numel() != k:
        raise ValueError(f"gemm shapes do not agree: resid {tuple(resid.shape)}, w {tuple(w.shape)}")
    if num_rows > GEMM_NORMED_MAX_TOKENS:
        raise ValueError(f"gemm_bf16_normed takes at most {GEMM_NORMED_MAX_TOKENS} rows, got {num_rows}")
    want = torch.bfloat16 if mode in (GEMM_OUT_BF16, GEMM_SWIGLU) else torch.float32
    _need(out, want, "out")
    if out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"output {tuple(out.shape)} does not match width {n}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    code = core().vx_gemm_bf16_normed(_p(resid), resid.stride(0), _p(norm_weight), float(eps), _p(w), _p(bias),
                                      _p(out), mode, num_rows, n, k, out.stride(0), splits, _p(status), _stream())
    if code == -2:
        return False
    if code == -1:
        raise KernelError(
            f"gemm_bf16_normed refuses resid {tuple(resid.shape)} w {tuple(w.shape)}: the inner size must "
            "be a multiple of 8, the row pitch of resid a multiple of 4 and the operands 16-byte aligned"
        )
    _check(code, "gemm_bf16_normed")
    return True


def gemm_bf16_add_mirrored(
    x: torch.Tensor,
    w: torch.Tensor,
    out: torch.Tensor,
    mirror: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
    splits: int,
) -> bool:
    """out[:num_rows] += x[:num_rows] @ w.T (float32) with the sums also written to ``mirror``:
    a copy of the rows that stays as it is while a later kernel adds to ``out`` again.  False
    (nothing launched) where the launch would not be split along K."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.float32, "out")
    if mirror.dtype != torch.float32 or mirror.dim() != 2 or mirror.stride(1) != 1 or mirror.shape[1] != out.shape[1]:
        raise TypeError("mirror must be float32 rows of the width of out")
    n, k = w.shape
    if x.shape[1] != k or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = core().vx_gemm_bf16_add_mirrored(_p(x), _p(w), _p(out), _p(mirror), num_rows, x.shape[0], n, k,
                                            out.stride(0), mirror.stride(0), splits, _p(status), _stream())
    if code in (-1, -4):
        return False
    _check(code, "gemm_bf16_add_mirrored")
    return True


# Steps of at most this many tokens can run the gated feed-forward as one kernel.
MLP_FUSED_MAX_TOKENS = 32


def mlp_fused(
    resid_in: torch.Tensor,
    norm_weight: torch.Tensor,
    eps: float,
    w_gate_up: torch.Tensor,
    w_down: torch.Tensor,
    resid_out: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
) -> bool:
    """resid_out[:num_rows] += w_down @ (silu(gate) * up) of rmsnorm(resid_in[:num_rows]) *
    norm_weight, in one kernel (see ``mlp_fused_kernel`` in gemm_bf16.cu): the norm is made on
    the spot, the activations stay on the SM, and the CTAs' shares of the sum over the inner
    width meet in ``resid_out`` by float32 reductions at the L2, whose order is not fixed.
    ``resid_in`` and ``resid_out`` are float32 rows and must not overlap (other CTAs add to
    the output while a CTA still reads its input).  False (nothing launched) when the sizes
    do not fit: more than ``MLP_FUSED_MAX_TOKENS`` rows, a width that is no multiple of 128 or
    too long for shared or tensor memory, an inner width that is no multiple of 64."""
    for name, t in (("resid_in", resid_in), ("resid_out", resid_out)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
            raise TypeError(f"{name} must be float32 rows on the device")
    _need(norm_weight, torch.float32, "norm_weight")
    _need(w_gate_up, torch.bfloat16, "w_gate_up")
    _need(w_down, torch.bfloat16, "w_down")
    width = resid_in.shape[1]
    inner = w_down.shape[1]
    if w_gate_up.shape != (2 * inner, width) or w_down.shape[0] != width or resid_out.shape[1] != width:
        raise ValueError(
            f"mlp_fused shapes do not agree: rows of {width}, gate|up {tuple(w_gate_up.shape)}, down {tuple(w_down.shape)}")
    if norm_weight.numel() != width:
        raise ValueError("mlp_fused: the norm weight has another width than the rows")
    if num_rows > MLP_FUSED_MAX_TOKENS or width % 128 or inner % 64 or resid_in.stride(0) % 4:
        return False
    if resid_in.data_ptr() == resid_out.data_ptr():
        raise ValueError("mlp_fused: resid_in and resid_out must be different buffers")
    code = core().vx_mlp_fused(_p(resid_in), resid_in.stride(0), _p(norm_weight), float(eps), _p(w_gate_up),
                               _p(w_down), _p(resid_out), resid_out.stride(0), num_rows, width, inner,
                               _p(status), _stream())
    if code in (-1, -2):
        return False
    _check(code, "mlp_fused")
    return True


def gemm_bf16_qkv_rope(
    x: Optional[torch.Tensor],
    resid: Optional[torch.Tensor],
    norm_weight: Optional[torch.Tensor],
    eps: float,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    status: torch.Tensor,
    splits: int,
) -> bool:
    """The QKV projection of heads of 128 dims with rotate-half RoPE and the cache write in its
    epilogue: rotated queries go to ``out`` [rows, (heads + 2 kv_heads) * 128] (its key and
    value columns are left as they are), rotated keys and the values into the paged caches at
    ``slots`` (None caches: no write).  The input is ``x`` (bfloat16) or, when ``resid`` is
    given, ``rmsnorm(resid) * norm_weight``.  False, with nothing launched, for shapes the
    kernel does not take (then project and rotate separately)."""
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16, "out")
    _need(positions, torch.int32, "positions")
    _need(slots, torch.int32, "slots")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    n, k = w.shape
    if n != (num_heads + 2 * num_kv_heads) * 128 or out.shape[1] != n or cos.shape[1] != 64:
        return False
    if num_rows > GEMM_NORMED_MAX_TOKENS:
        return False
    if resid is not None:
        if resid.dtype != torch.float32 or resid.stride(1) != 1 or resid.shape[1] != k:
            raise TypeError("resid must be float32 rows as wide as the weight")
        _need(norm_weight, torch.float32, "norm_weight")
    else:
        _need(x, torch.bfloat16, "x")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    write = k_cache is not None
    if write:
        _need(k_cache, torch.bfloat16, "k_cache")
        _need(v_cache, torch.bfloat16, "v_cache")
        if k_cache.shape[2] != num_kv_heads or k_cache.shape[3] != 128:
            return False
    num_slots = k_cache.shape[0] * k_cache.shape[1] if write else 0
    code = core().vx_gemm_bf16_qkv_rope(
        _p(x), 0 if x is None else x.shape[0], _p(resid), 0 if resid is None else resid.stride(0),
        _p(norm_weight), float(eps), _p(w), _p(bias), _p(out), num_rows, k, out.stride(0), splits,
        _p(positions), _p(cos), _p(sin), cos.shape[0], _p(slots), _p(k_cache), _p(v_cache), num_slots,
        num_heads, num_kv_heads, _p(status), _stream())
    if code in (-1, -2):
        return False
    _check(code, "gemm_bf16_qkv_rope")
    return True


def cast_bf16_to_f32(src: torch.Tensor, out: torch.Tensor, count: int) -> None:
    _need(src, torch.bfloat16, "src")
    _need(out, torch.float32, "out")
    _check(core().vx_cast_bf16_to_f32(_p(src), _p(out), count, _stream()), "cast")


# ------------------------------------------------------------------------------------------
ATTN_F32, ATTN_BF16_WIDE, ATTN_BF16_NARROW, ATTN_BF16_TC = 0, 1, 2, 3


def tile_rows(kind: int) -> int:
    return {ATTN_BF16_WIDE: 64, ATTN_BF16_TC: 128}.get(kind, 16)


def attention(
    kind: int,
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    q_len: torch.Tensor,
    kv_len: torch.Tensor,
    items: torch.Tensor,
    num_items: int,
    partial_o: Optional[torch.Tensor],
    partial_lse: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: Optional[int],
    softmax_scale: float,
    merge_items: Optional[torch.Tensor] = None,
    split_counters: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    cluster: int = 1,
    layout_checked: bool = False,
    keep_first: int = 0,
    softcap: float = 0.0,
    distance_bias: Optional[tuple] = None,
    chunk: int = 0,
    sink_zero: bool = False,
    row_scale: Optional[torch.Tensor] = None,
) -> None:
    """Run ``num_items`` work items (see attention.cu for their layout) of one kernel family.

    ``layout_checked``: the caller has passed these same index and scratch tensors before (the
    step's layout is shared by all layers); only q, out and the caches are checked again.

    With ``merge_items`` and ``split_counters`` (int32, zero, one per merge item and KV head)
    the bfloat16 families merge split key ranges themselves: the last split to finish does it.
    ``cluster`` (1, 2, 4 or 8; narrow bfloat16 family) CTAs share every item as a thread-block
    cluster: each takes a run of the item's key tiles and they merge through distributed shared
    memory.  For the tensor-memory family 2 asks for two CTAs on an SM whatever the grid's size
    (the caller knows that the items' key ranges are long).  ``keep_first`` (with a window): keys
    0 .. keep_first - 1 stay visible to every later query.

    Changes to a score ``s = (q . k) * softmax_scale`` before the softmax (not in the
    tensor-memory family): ``row_scale`` (float32 table over positions): ``s *= row_scale[pos]``;
    ``softcap`` c > 0: ``s = c tanh(s / c)``; ``distance_bias`` (r1, r2), float32 per query head:
    ``s -= r1 ln(1 + r2 (pos - n))``; ``chunk`` c > 0: a query at ``pos`` sees keys from
    ``floor(pos / c) * c`` on; ``sink_zero``: one more term of score 0 and no value in every
    row's denominator (layers without window or chunk).
    """
    want = torch.float32 if kind == ATTN_F32 else torch.bfloat16
    _need(q, want, "q")
    _need(out, want, "out")
    _need(k_cache, want, "k_cache")
    _need(v_cache, want, "v_cache")
    if k_cache.shape[2] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not match {num_kv_heads} x {head_dim}")
    if not layout_checked:
        for name, t in (("block_tables", block_tables), ("q_start", q_start), ("q_len", q_len),
                        ("kv_len", kv_len), ("items", items)):
            _need(t, torch.int32, name)
        if num_heads % num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if partial_o is not None:
            _need(partial_o, torch.float32, "partial_o")
            _need(partial_lse, torch.float32, "partial_lse")
        if split_counters is not None:
            _need(split_counters, torch.int32, "split_counters")
            _need(merge_items, torch.int32, "merge_items")
    lib = attention_lib(head_dim)
    r1 = r2 = None
    if distance_bias is not None:
        r1, r2 = distance_bias
        _need(r1, torch.float32, "distance_bias r1")
        _need(r2, torch.float32, "distance_bias r2")
        if r1.numel() != num_heads or r2.numel() != num_heads:
            raise ValueError("the distance bias needs two numbers per query head")
    if row_scale is not None:
        _need(row_scale, torch.float32, "row_scale")
    _check(
        lib.vx_attention_scored(kind, _p(q), _p(out), _p(k_cache), _p(v_cache), _p(block_tables),
                                _p(q_start), _p(q_len), _p(kv_len), _p(items), num_items,
                                _p(status if status is not None else _attention_status()),
                                _p(partial_o), _p(partial_lse), _p(merge_items), _p(split_counters),
                                q.shape[1], out.shape[1],
                                block_tables.shape[1], num_kv_heads, num_heads // num_kv_heads,
                                k_cache.shape[1], k_cache.shape[0], int(window or 0), float(softmax_scale),
                                int(cluster), int(keep_first or 0), float(softcap or 0.0), _p(r1), _p(r2),
                                int(chunk or 0), 1 if sink_zero else 0, _p(row_scale),
                                0 if row_scale is None else row_scale.numel(), _stream()),
        "attention",
    )


def attention_has_tc(head_dim: int) -> bool:
    """Whether prompt portions of this head size run on the tensor-memory (tcgen05) family."""
    return bool(attention_lib(head_dim).vx_attn_has_tc())


def narrow_attention_slots(head_dim: int) -> int:
    """Work items of the narrow bfloat16 family that one SM holds at a time."""
    return int(attention_lib(head_dim).vx_attn_narrow_ctas_per_sm())


def max_attention_cluster(head_dim: int) -> int:
    return int(attention_lib(head_dim).vx_attn_max_cluster())


def attention_cluster_limits(head_dim: int) -> tuple:
    """((cluster size, clusters of that size the device holds at a time), ...), largest first."""
    _require_cuda()
    lib = attention_lib(head_dim)
    limits = []
    size = max_attention_cluster(head_dim)
    while size >= 2:
        count = int(lib.vx_attn_narrow_max_active_clusters(size))
        if count < 0:
            raise KernelError(f"cluster occupancy query for size {size}: CUDA error {-count}")
        limits.append((size, count))
        size //= 2
    return tuple(limits)


_default_status = None


def _attention_status() -> torch.Tensor:
    """A status word for callers that pass none (bounded waits need somewhere to report)."""
    global _default_status
    if _default_status is None:
        _default_status = torch.zeros(4, dtype=torch.int32, device="cuda")
    return _default_status


def attention_merge(
    out: torch.Tensor,
    q_start: torch.Tensor,
    merge_items: torch.Tensor,
    num_items: int,
    partial_o: torch.Tensor,
    partial_lse: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    max_rows: int = 64,
    sinks: Optional[torch.Tensor] = None,
) -> None:
    """Combine the splits of the merge items; ``max_rows`` bounds the rows of any item.
    ``sinks`` (float32, one per query head): exp(sink) joins every row's softmax denominator,
    with no key and no value."""
    _need(merge_items, torch.int32, "merge_items")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks")
        if sinks.numel() != num_heads:
            raise ValueError("one sink per query head is needed")
    lib = attention_lib(head_dim)
    _check(
        lib.vx_attention_merge(_code(out.dtype), _p(out), _p(q_start), _p(merge_items), num_items,
                               max_rows, _p(partial_o), _p(partial_lse), out.shape[1], num_kv_heads,
                               num_heads // num_kv_heads, _p(sinks), _stream()),
        "attention_merge",
    )


# ------------------------------------------------------------------------------------------
# Scratch of the sampling kernel per device: the segments' best entries and the rows' arrival
# counters (zero between launches; the kernel puts them back).
_sample_scratch: dict = {}


def _sample_scratch_for(device: torch.device, num_rows: int, vocab: int):
    segments = core().vx_sample_segments(num_rows, vocab)
    if segments <= 1:
        return None, None
    key = (device.type, device.index)
    held = _sample_scratch.get(key)
    if held is None or held[0].shape[0] < num_rows * segments or held[1].shape[0] < num_rows:
        rows = max(num_rows, 64)
        held = (
            torch.zeros((rows * 64, 2), dtype=torch.int32, device=device),
            torch.zeros(rows, dtype=torch.int32, device=device),
        )
        _sample_scratch[key] = held
    return held


def sample(
    logits: torch.Tensor,
    num_rows: int,
    temperature: Optional[torch.Tensor],
    seeds: Optional[torch.Tensor],
    draw_index: Optional[torch.Tensor],
    threshold: Optional[torch.Tensor],
    out: torch.Tensor,
    history: Optional[torch.Tensor] = None,
    history_slots: Optional[torch.Tensor] = None,
    history_lengths: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> None:
    """One token per row: argmax where temperature is 0 (or None), else the exponential race.

    With ``history`` (int32 [slots, width]) the token of row r is also stored at
    ``history[history_slots[r], history_lengths[r]]``.  With ``status`` (the device status
    word) its first entry is copied to ``out[num_rows]``, so ``out`` needs one entry more."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    if out.numel() < num_rows + (0 if status is None else 1):
        raise ValueError("out is too short for the rows (and the status word)")
    if temperature is not None:
        _need(temperature, torch.float32, "temperature")
        _need(seeds, torch.int64, "seeds")
        _need(draw_index, torch.int32, "draw_index")
    partial, counters = _sample_scratch_for(logits.device, num_rows, logits.shape[1])
    _check(
        core().vx_sample(_p(logits), num_rows, logits.shape[1], logits.stride(0), _p(temperature),
                         _p(seeds), _p(draw_index), _p(threshold), _p(out), _p(history),
                         0 if history is None else history.stride(0), _p(history_slots),
                         _p(history_lengths), _p(partial), _p(counters), _p(status), _stream()),
        "sample",
    )


def filter_threshold(
    logits: torch.Tensor,
    num_rows: int,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    threshold: torch.Tensor,
    kind: int = 0,
) -> None:
    """threshold[r]: the smallest scaled logit that is a top-k / top-p candidate of row r.

    ``kind`` picks the kernel: 0 a cluster of eight CTAs per row where the row fits their
    registers (196,608 entries) and one CTA per row otherwise, 1 always one CTA per row, 2 the
    cluster kernel or an error.  Both give the same threshold bit for bit."""
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k")
    _need(top_p, torch.float32, "top_p")
    _need(threshold, torch.float32, "threshold")
    _check(
        core().vx_filter_threshold(_p(logits), num_rows, logits.shape[1], logits.stride(0),
                                   _p(temperature), _p(top_k), _p(top_p), _p(threshold), kind, _stream()),
        "filter_threshold",
    )


def apply_penalties(
    logits: torch.Tensor,
    num_rows: int,
    history: torch.Tensor,
    slots: torch.Tensor,
    lengths: torch.Tensor,
    counts: torch.Tensor,
    repetition: torch.Tensor,
    presence: torch.Tensor,
    frequency: torch.Tensor,
) -> None:
    _need(logits, torch.float32, "logits")
    _need(history, torch.int32, "history")
    _need(slots, torch.int32, "slots")
    _need(lengths, torch.int32, "lengths")
    _need(counts, torch.int32, "counts")
    _check(
        core().vx_apply_penalties(_p(logits), num_rows, logits.shape[1], logits.stride(0),
                                  _p(history), history.stride(0), _p(slots), _p(lengths),
                                  _p(counts), _p(repetition), _p(presence), _p(frequency),
                                  _stream()),
        "apply_penalties",
    )


# ------------------------------------------------------------------------------------------
# Recurrent mixers, expert feed-forwards and the row-wise kernels around them (csrc/sequence.cu,
# csrc/routed.cu).  Tensors may be column ranges of wider buffers: a row pitch is passed.
ACT_NONE, ACT_SILU, ACT_GELU_TANH, ACT_RELU_SQUARED, ACT_TANH = 0, 1, 2, 3, 4


def _pitched(t: torch.Tensor, name: str) -> int:
    """Row pitch (elements) of a 2-D tensor whose rows are contiguous."""
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{name} must be 2-D with contiguous rows")
    return t.stride(0)


def pair_rope_cache_write(qkv, positions, cos, sin, slots, k_cache, v_cache, num_tokens, num_heads, num_kv_heads,
                          head_dim, rotary_dim, status) -> None:
    """Neighbouring pairs (2i, 2i + 1) of the first ``rotary_dim`` dims of every q and k head turn
    by the tabulated angles (q in place); k and v go to the cache at ``slots``.  The rows of
    ``qkv`` hold q | k | v and possibly further columns behind them."""
    stride = _pitched(qkv, "qkv")
    if qkv.shape[1] < (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv rows are narrower than the heads")
    write = k_cache is not None
    if write:
        _need(k_cache, qkv.dtype, "k_cache")
        _need(v_cache, qkv.dtype, "v_cache")
    if rotary_dim > 0:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if cos.shape[1] != rotary_dim // 2 or rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError("cos/sin tables do not match the rotary width")
    _check(
        mixers().vx_pair_rope_cache_write(
            _p(qkv), _code(qkv.dtype), stride, _p(positions), _p(cos) if rotary_dim > 0 else None,
            _p(sin) if rotary_dim > 0 else None, _p(slots), _p(k_cache), _p(v_cache), num_tokens, num_heads,
            num_kv_heads, head_dim, rotary_dim, cos.shape[0] if rotary_dim > 0 else 0,
            k_cache.shape[0] * k_cache.shape[1] if write else 0, 1 if write else 0, _p(status), _stream()),
        "pair_rope_cache_write",
    )


def head_gate(out, logits, num_tokens, num_heads, head_dim) -> None:
    """out[t, h, :] *= sigmoid(logits[t, h])."""
    _check(mixers().vx_head_gate(_p(out), _code(out.dtype), _pitched(out, "out"), _p(logits),
                                 _pitched(logits, "logits"), num_tokens, num_heads, head_dim, _stream()),
           "head_gate")


def conv_tokens(x, weight, bias, state, out, q_start, q_len, seq_slots, num_seqs, num_tokens, act) -> None:
    """Causal convolution per channel over each sequence's tokens and the update of its state.

    ``x`` [tokens, channels] (a column range is fine), ``weight`` float32 [channels, taps] with
    the last column the current token's, ``state`` float32 [slots, (taps - 1) * channels]: the
    last taps - 1 inputs of each slot's sequence.  ``out`` float32 [tokens, channels]."""
    _need(weight, torch.float32, "conv weight")
    _need(bias, torch.float32, "conv bias")
    channels, taps = weight.shape
    if x.shape[1] != channels or out.shape[1] != channels or out.dtype != torch.float32:
        raise ValueError("conv_tokens: widths do not agree")
    if state.dtype != torch.float32 or state.shape[1] < (taps - 1) * channels:
        raise ValueError("conv_tokens: the state is too small")
    _check(
        mixers().vx_conv_tokens(_p(x), _code(x.dtype), _pitched(x, "x"), channels, taps, _p(weight), _p(bias),
                                _p(state), _pitched(state, "state"), _p(out), _pitched(out, "out"), _p(q_start),
                                _p(q_len), _p(seq_slots), num_seqs, max(1, min(64, num_tokens)), act, _stream()),
        "conv_tokens",
    )


def rglru_gates(u, w_a_t, b_a, w_i_t, b_i, lam, decay_scale, a_out, b_out, num_tokens, w_a=None, w_i=None) -> None:
    """Decay and gated input of S <- a S + b from u float32 [tokens, width]; the gate matrices are
    block-diagonal, stored transposed [blocks, in, out], all float32.  ``w_a``, ``w_i``: the same
    matrices [blocks, out, in], which a step of a few tokens reads instead (a warp per output)."""
    blocks, part, _ = w_a_t.shape
    for name, t in (("w_a_t", w_a_t), ("b_a", b_a), ("w_i_t", w_i_t), ("b_i", b_i), ("lam", lam)):
        _need(t, torch.float32, name)
    if w_a is not None:
        _need(w_a, torch.float32, "w_a")
        _need(w_i, torch.float32, "w_i")
    _check(
        mixers().vx_rglru_gates(_p(u), _pitched(u, "u"), blocks * part, blocks, _p(w_a_t), _p(b_a), _p(w_i_t),
                                _p(b_i), _p(lam), float(decay_scale), _p(a_out), _p(b_out), _pitched(a_out, "a_out"),
                                num_tokens, _p(w_a), _p(w_i), _stream()),
        "rglru_gates",
    )


def rglru_scan_scratch(num_tokens: int, num_seqs: int, width: int) -> int:
    """float32 entries of scratch that ``rglru_scan`` needs to run a step's long portions in
    chunks."""
    chunk = int(mixers().vx_rglru_chunk_rows())
    return (2 * (num_tokens // chunk + num_seqs + 1) + num_seqs) * width


def rglru_scan(a_in, b_in, y, state, out, q_start, q_len, seq_slots, num_seqs, y_act, scratch=None,
               num_tokens=0) -> None:
    """S <- a S + b over every sequence's tokens from the state of its slot (float32
    [slots, width]); out = S * act(y).  With ``scratch`` (float32, ``rglru_scan_scratch`` entries)
    and ``num_tokens`` (the step's tokens) a long step runs in chunks of tokens side by side."""
    width = a_in.shape[1]
    if scratch is not None:
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < rglru_scan_scratch(num_tokens, num_seqs, width):
            raise ValueError("rglru_scan: the scratch is too small")
    _check(
        mixers().vx_rglru_scan(_p(a_in), _p(b_in), _pitched(a_in, "a_in"), _p(y), _code(y.dtype), _pitched(y, "y"),
                               width, _p(state), _pitched(state, "state"), _p(out), _pitched(out, "out"),
                               _p(q_start), _p(q_len), _p(seq_slots), num_seqs, y_act, _p(scratch), int(num_tokens),
                               _stream()),
        "rglru_scan",
    )


def ssd_scan_scratch(num_tokens: int, num_seqs: int, heads: int, state_size: int, value_dim: int) -> int:
    """float32 entries of scratch that ``ssd_scan`` needs to run a step's long portions in chunks."""
    chunk = int(mixers().vx_ssd_chunk_rows())
    return (num_tokens // chunk + num_seqs + 1) * heads * (state_size * value_dim + 1)


def ssd_scan(xbc, dt, dt_bias, a_log, d_skip, state, y_out, heads, groups, state_size, value_dim, q_start, q_len,
             seq_slots, num_seqs, scratch=None, num_tokens=0) -> None:
    """Per head: S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + D x with dt = softplus(dt +
    dt_bias); ``xbc`` float32 rows hold x | B | C, ``state`` float32 [slots, heads * N * P].  With
    ``scratch`` (float32, ``ssd_scan_scratch`` entries) and ``num_tokens`` (the step's tokens) a
    long step runs in chunks of tokens side by side."""
    if scratch is not None:
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < ssd_scan_scratch(num_tokens, num_seqs, heads, state_size, value_dim):
            raise ValueError("ssd_scan: the scratch is too small")
    _check(
        mixers().vx_ssd_scan(_p(xbc), _pitched(xbc, "xbc"), _p(dt), _code(dt.dtype), _pitched(dt, "dt"),
                             _p(dt_bias), _p(a_log), _p(d_skip), _p(state), _pitched(state, "state"), _p(y_out),
                             _pitched(y_out, "y_out"), heads, groups, state_size, value_dim, _p(q_start), _p(q_len),
                             _p(seq_slots), num_seqs, _p(scratch), int(num_tokens), _stream()),
        "ssd_scan",
    )


def gated_group_norm(y, z, weight, eps, parts, out, num_tokens, gate_after=False) -> None:
    """out = (y * silu(z)) divided, in ``parts`` equal parts, by each part's RMS, times weight; with
    ``gate_after``: y divided by each part's RMS, times weight, times sigmoid(z)."""
    inner = weight.numel()
    _check(
        mixers().vx_gated_group_norm(_p(y), _pitched(y, "y"), _p(z), _code(z.dtype), _pitched(z, "z"), _p(weight),
                                     float(eps), inner, parts, _p(out), _pitched(out, "out"), num_tokens,
                                     1 if gate_after else 0, _stream()),
        "gated_group_norm",
    )


def delta_rule_packed_width(heads: int, key_dim: int, value_dim: int) -> int:
    """float32 values per token of the scratch rows ``delta_rule_scan`` wants."""
    width = mixers().vx_delta_rule_packed_width(heads, key_dim, value_dim)
    if width < 0:
        raise KernelError(f"delta_rule_scan refuses a key size of {key_dim} (at most 512)")
    return width


def delta_rule_chunk_scratch(num_tokens: int, num_seqs: int, heads: int, key_dim: int, value_dim: int) -> int:
    """float32 values of scratch with which ``delta_rule_scan`` runs long steps in chunks side by side."""
    return int(mixers().vx_delta_rule_chunk_scratch(num_tokens, num_seqs, heads, key_dim, value_dim))


def delta_rule_scan(r, k, v, a, w, w0, a_bias, decay, key_eps, state, out, heads, key_dim, value_dim, q_start, q_len,
                    seq_slots, num_seqs, num_tokens, packed, status, chunk_scratch=None) -> None:
    """The generalized delta rule over each sequence's tokens (csrc/sequence.cu).  ``r``, ``k``,
    ``v``, ``a`` are column ranges of one projection buffer [tokens, *] (heads x key_dim, value_dim for
    v), ``w`` the decay's logits [tokens, heads * key_dim]; ``w0``, ``a_bias`` float32 [heads *
    key_dim]; ``state`` float32, a row per state slot holding [heads, value_dim, key_dim]; ``out``
    float32 [tokens, heads * value_dim]; ``packed`` float32 scratch [at least tokens,
    delta_rule_packed_width(...)]: the tokens' vectors as the scan reads them (the kernels lay it
    out head by head).  ``chunk_scratch`` (float32, ``delta_rule_chunk_scratch`` values for the step's
    tokens and sequences at least): steps of 512 tokens and more then run in chunks of 256 tokens side
    by side; a token's result then depends, within float32 rounding, on where its chunk began."""
    stride = _pitched(r, "r")
    if _pitched(k, "k") != stride or _pitched(v, "v") != stride or _pitched(a, "a") != stride:
        raise ValueError("delta_rule_scan: r, k, v and a are columns of one buffer")
    if w.dtype != r.dtype or out.dtype != torch.float32 or state.dtype != torch.float32:
        raise TypeError("delta_rule_scan: logits in the compute dtype, state and out float32")
    _need(w0, torch.float32, "w0")
    _need(a_bias, torch.float32, "a_bias")
    _need(packed, torch.float32, "packed")
    _need(status, torch.int32, "status")
    if chunk_scratch is not None:
        _need(chunk_scratch, torch.float32, "chunk_scratch")
    if state.shape[1] < heads * key_dim * value_dim or state.stride(1) != 1:
        raise ValueError("delta_rule_scan: the state row is too small")
    if packed.shape[0] < num_tokens or packed.shape[1] != delta_rule_packed_width(heads, key_dim, value_dim):
        raise ValueError("delta_rule_scan: the scratch rows do not fit")
    code = mixers().vx_delta_rule_scan(
        _p(r), _p(k), _p(v), _p(a), _code(r.dtype), stride, _p(w), _pitched(w, "w"), _p(w0), _p(a_bias),
        float(decay), float(key_eps), _p(packed), packed.shape[0], _p(state), state.stride(0), _p(out),
        _pitched(out, "out"), heads,
        key_dim, value_dim, _p(q_start), _p(q_len), _p(seq_slots), num_seqs, num_tokens, _p(chunk_scratch),
        0 if chunk_scratch is None else chunk_scratch.numel(), _p(status), _stream())
    if code == -1:
        raise KernelError(f"delta_rule_scan refuses a key size of {key_dim} (at most 512)")
    _check(code, "delta_rule_scan")


def dual_norm_mean(a, b, w_a, w_b, eps, scale, num_tokens, resid=None, out=None) -> None:
    """scale * (rms_norm(a) * w_a + rms_norm(b) * w_b): added to ``resid`` (float32) or written
    to ``out``."""
    _need(a, a.dtype, "a")
    _need(b, a.dtype, "b")
    if (resid is None) == (out is None):
        raise ValueError("dual_norm_mean writes either into the stream or to a buffer")
    _check(
        mixers().vx_dual_norm_mean(_p(a), _p(b), _code(a.dtype), _p(w_a), _p(w_b), float(eps), float(scale),
                                   a.shape[1], _p(resid), _p(out), num_tokens, _stream()),
        "dual_norm_mean",
    )


def act_rows(x, out, num_tokens, kind) -> None:
    """out = act(x) column by column; both may be column ranges of wider buffers."""
    _check(
        mixers().vx_act_rows(_p(x), _code(x.dtype), _pitched(x, "x"), _p(out), _pitched(out, "out"), out.shape[1],
                             num_tokens, kind, _stream()),
        "act_rows",
    )


def residual_add(resid, delta, num_tokens) -> None:
    """resid[:n] += delta[:n] in float32."""
    _need(resid, torch.float32, "resid")
    _need(delta, delta.dtype, "delta")
    _check(mixers().vx_residual_add(_p(resid), _p(delta), _code(delta.dtype), num_tokens * resid.shape[1], _stream()),
           "residual_add")


def gated_rows_add(resid, x, logit, num_tokens) -> None:
    """resid[t, :] += sigmoid(logit[t]) * x[t, :]; ``logit`` is one column of a wider buffer."""
    _need(resid, torch.float32, "resid")
    _need(x, x.dtype, "x")
    _check(
        mixers().vx_gated_rows_add(_p(resid), _p(x), _p(logit), _code(x.dtype), _pitched(logit, "logit"),
                                   resid.shape[1], num_tokens, _stream()),
        "gated_rows_add",
    )


def table_experts(h, ids, fed, table, w_up, w_down, resid, num_tokens, status) -> None:
    """Every token's experts, named by row ``ids[t]`` of ``table`` [vocab, top]: the mean of
    ``W_down[e] relu(W_up[e] h)^2`` over them is added to ``resid``.  ``w_up`` [experts, ff,
    width], ``w_down`` [experts, width, ff]."""
    _need(table, torch.int32, "table")
    _need(ids, torch.int32, "ids")
    _need(w_up, h.dtype, "w_up")
    _need(w_down, h.dtype, "w_down")
    _need(resid, torch.float32, "resid")
    experts, ff, width = w_up.shape
    vocab, top = table.shape
    _check(
        mixers().vx_table_experts(_p(h), _code(h.dtype), _pitched(h, "h"), _p(ids), _p(fed),
                                  0 if fed is None else fed.numel(), _p(table), vocab, top, experts, _p(w_up),
                                  _p(w_down), width, ff, _p(resid), num_tokens, _p(status), _stream()),
        "table_experts",
    )


def table_experts_rows(h, ids, fed, table, w_up, w_down, act, resid, num_tokens, status) -> bool:
    """``table_experts`` as two launches whose blocks each take some rows of one (token, expert)
    pair's projection: ``act`` float32 [tokens * top * ff] holds the activations in between.
    False (nothing done): a row or a token's activations do not fit a block's shared memory."""
    experts, ff, width = w_up.shape
    vocab, top = table.shape
    if width * 4 > 48 * 1024 or top * ff * 4 > 48 * 1024:
        return False
    _need(table, torch.int32, "table")
    _need(ids, torch.int32, "ids")
    _need(w_up, h.dtype, "w_up")
    _need(w_down, h.dtype, "w_down")
    _need(resid, torch.float32, "resid")
    _need(act, torch.float32, "act")
    if act.numel() < num_tokens * top * ff:
        raise ValueError("table_experts_rows: the activation buffer is too small")
    _check(
        mixers().vx_table_experts_rows(_p(h), _code(h.dtype), _pitched(h, "h"), _p(ids), _p(fed),
                                       0 if fed is None else fed.numel(), _p(table), vocab, top, experts, _p(w_up),
                                       _p(w_down), width, ff, _p(act), _p(resid), num_tokens, _p(status), _stream()),
        "table_experts_rows",
    )
    return True


def grouped_places(num_tokens: int, top: int, experts: int) -> int:
    """Places (rows of the ordered pairs, every expert's run padded to whole tiles) that
    ``table_experts_grouped`` needs for a step."""
    tile = int(mixers().vx_grouped_tile_rows())
    return -(-(num_tokens * top + experts * (tile - 1)) // tile) * tile


def table_experts_grouped(h, ids, fed, table, w_up, w_down, route, act, rows, resid, num_tokens, status) -> bool:
    """``table_experts`` for long bfloat16 steps: the pairs ordered by expert, both projections as
    tiled tensor-core products.  ``route`` int32 scratch, ``act`` bfloat16 [places, ff],
    ``rows`` float32 [places, width] (see ``grouped_places``).  False: sizes it does not take."""
    experts, ff, width = w_up.shape
    vocab, top = table.shape
    if h.dtype != torch.bfloat16 or width % 8 or ff % 8 or _pitched(h, "h") % 8 or experts * 12 > 48 * 1024:
        return False
    places = grouped_places(num_tokens, top, experts)
    tile = int(mixers().vx_grouped_tile_rows())
    if (route.numel() < places // tile + places + num_tokens * top or act.shape[0] < places or rows.shape[0] < places
            or act.shape[1] != ff or rows.shape[1] != width):
        raise ValueError("table_experts_grouped: the scratch buffers are too small")
    _need(route, torch.int32, "route")
    _need(act, torch.bfloat16, "act")
    _need(rows, torch.float32, "rows")
    _need(resid, torch.float32, "resid")
    _check(
        mixers().vx_table_experts_grouped(_p(h), _pitched(h, "h"), _p(ids), _p(fed), 0 if fed is None else fed.numel(),
                                          _p(table), vocab, top, experts, _p(w_up), _p(w_down), width, ff, _p(route),
                                          places, _p(act), ff, _p(rows), _p(resid), num_tokens, _p(status), _stream()),
        "table_experts_grouped",
    )
    return True


_library_grouped_refused = False


def has_library_grouped_product() -> bool:
    """Whether torch offers a grouped matrix product with the groups' ends on the device (and
    has not refused a call of this process)."""
    return hasattr(torch, "_grouped_mm") and not _library_grouped_refused


def table_experts_library(h, ids, fed, table, w_up, w_down, route, run_ends, a_rows, resid, num_tokens, status) -> bool:
    """``table_experts`` for long bfloat16 steps with the two products as the library's grouped
    product (one launch each over all experts, the runs' ends read on the device): this
    package's kernels order the pairs by expert and gather the rows (``vx_route_and_gather``),
    square the positive parts, and sum a token's pairs into the stream.  ``route`` int32 scratch
    as for ``table_experts_grouped``, ``run_ends`` int32 [experts], ``a_rows`` bfloat16
    [places, width].  False: sizes it does not take, or no such product in this torch."""
    experts, ff, width = w_up.shape
    vocab, top = table.shape
    if (not has_library_grouped_product() or h.dtype != torch.bfloat16 or width % 16 or ff % 16
            or _pitched(h, "h") % 8 or experts * 12 > 48 * 1024):
        return False
    places = grouped_places(num_tokens, top, experts)
    tile = int(mixers().vx_grouped_tile_rows())
    if route.numel() < places // tile + places + num_tokens * top or a_rows.shape[0] < places or a_rows.shape[1] != width:
        raise ValueError("table_experts_library: the scratch buffers are too small")
    _need(route, torch.int32, "route")
    _need(run_ends, torch.int32, "run_ends")
    _need(a_rows, torch.bfloat16, "a_rows")
    _need(resid, torch.float32, "resid")
    _check(
        mixers().vx_route_and_gather(_p(h), _pitched(h, "h"), _p(ids), _p(fed), 0 if fed is None else fed.numel(),
                                     _p(table), vocab, top, experts, width, _p(route), places, _p(run_ends),
                                     _p(a_rows), num_tokens, _p(status), _stream()),
        "route_and_gather",
    )
    global _library_grouped_refused
    try:
        up = torch._grouped_mm(a_rows[:places], w_up.transpose(1, 2), offs=run_ends)
        note_library_launch("library_grouped_gemm")
        act_rows(up, up, places, ACT_RELU_SQUARED)
        down = torch._grouped_mm(up, w_down.transpose(1, 2), offs=run_ends)
        note_library_launch("library_grouped_gemm")
    except (RuntimeError, TypeError, ValueError, NotImplementedError):
        # The library does not take these sizes (or this build has no kernel for them): nothing
        # has been added to the stream yet, and the caller's own kernels take over for good.
        _library_grouped_refused = True
        return False
    _check(mixers().vx_gather_pairs(_p(down), _p(route), places, top, width, _p(resid), num_tokens, _stream()),
           "gather_pairs")
    return True


# ------------------------------------------------------------------------------------------
# The ``heads`` library.
def norm_shift(resid, weight, eps, out, num_tokens, q_start, q_len, seq_slots, num_seqs, weight2=None, out2=None,
               shift=None, state=None) -> None:
    """``out = h`` with ``h = resid / rms(resid) * weight`` per row, or, with ``shift`` (float32
    [width]) and ``state`` (float32, a row per state slot), ``h + (h_before - h) * shift`` where
    ``h_before`` is the same norm of the request's previous token (from the row above, or from
    the state row for a portion's first row; the portion's last ``h`` goes into the state row).
    ``weight2`` / ``out2``: a second output ``resid / rms(resid) * weight2`` from the same
    statistic."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    width = resid.shape[1]
    if weight2 is not None:
        _need(weight2, torch.float32, "weight2")
        _need(out2, out.dtype, "out2")
    if shift is not None:
        _need(shift, torch.float32, "shift")
        if state is None or state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < width:
            raise ValueError("token shift needs a float32 state row of at least the width per slot")
    _check(heads().vx_norm_shift(_p(resid), resid.stride(0), width, float(eps), _p(weight), _p(weight2), _p(shift),
                                 _p(state), 0 if state is None else state.stride(0), _p(out), _p(out2),
                                 _code(out.dtype), _p(q_start), _p(q_len), _p(seq_slots), int(num_seqs),
                                 int(num_tokens), _stream()),
           "norm_shift")


def add_rows(resid, a, b, num_tokens, scale_a: float = 1.0, scale_b: float = 1.0) -> None:
    """resid[:num_tokens] += scale_a * a (+ scale_b * b), float32 sums; a and b in the compute dtype,
    same row width."""
    _need(resid, torch.float32, "resid")
    _need(a, a.dtype, "a")
    if b is not None:
        _need(b, a.dtype, "b")
    _check(heads().vx_add_rows(_p(resid), _p(a), _p(b), _code(a.dtype), num_tokens * resid.shape[1],
                               float(scale_a), float(scale_b), _stream()),
           "add_rows")


def norm_conv(resid, weight, eps, conv_weight_t, state, out, num_tokens, q_start, q_len, seq_slots, num_seqs) -> None:
    """``out = h + conv(h)`` with ``h = resid / rms(resid) * weight`` per row and ``conv(h)_t = sum_j
    taps[j] * h_(t - taps + 1 + j)`` over a request's own tokens (zeros before its first).
    ``conv_weight_t`` float32 [taps, width]: the taps, the current token's last.  ``state`` float32,
    a row per state slot: the request's last taps - 1 values of h, oldest first; read for a
    portion's first rows and then rewritten."""
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(conv_weight_t, torch.float32, "conv_weight_t")
    width = resid.shape[1]
    taps = conv_weight_t.shape[0]
    if conv_weight_t.shape[1] != width or out.shape[1] != width or not out.is_contiguous():
        raise ValueError("norm_conv: widths do not agree")
    if taps > 1 and (state is None or state.dtype != torch.float32 or state.stride(-1) != 1
                     or state.shape[1] < (taps - 1) * width):
        raise ValueError("norm_conv needs a float32 state row of (taps - 1) * width values per slot")
    code = heads().vx_norm_conv(_p(resid), resid.stride(0), width, float(eps), _p(weight), _p(conv_weight_t), taps,
                                _p(state), 0 if state is None else state.stride(0), _p(out), _code(out.dtype),
                                _p(q_start), _p(q_len), _p(seq_slots), int(num_seqs), int(num_tokens), _stream())
    if code == -1:
        raise KernelError(f"norm_conv refuses {taps} taps (1 to 8)")
    _check(code, "norm_conv")


def diff_prepare(proj, qbuf, positions, cos, sin, q_norm, k_norm, eps, slots, k_cache, v_cache, num_tokens,
                 num_heads, num_kv_heads, dim, vdim, head_dim, rotary_dim, status) -> None:
    """Differential attention's way into the attention kernels (see csrc/heads.cu): per (head,
    map) RMS norm and rotation of q and k; q into ``qbuf`` [T, 2 H * head_dim], k of both maps side
    by side and v into their cache rows."""
    stride = _pitched(proj, "proj")
    write = k_cache is not None
    if rotary_dim > 0:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if cos.shape[1] != rotary_dim // 2:
            raise ValueError("cos/sin tables do not match the rotary width")
    _check(heads().vx_diff_prepare(
        _p(proj), _code(proj.dtype), stride, _p(qbuf), qbuf.stride(0), _p(positions),
        _p(cos) if rotary_dim > 0 else None, _p(sin) if rotary_dim > 0 else None, _p(q_norm), _p(k_norm),
        float(eps), _p(slots), _p(k_cache), _p(v_cache), num_tokens, num_heads, num_kv_heads, dim, vdim,
        head_dim, rotary_dim, cos.shape[0] if rotary_dim > 0 else 0,
        k_cache.shape[0] * k_cache.shape[1] if write else 0, 1 if write else 0, _p(status), _stream()),
        "diff_prepare")


def diff_combine(attn, gate, out, num_tokens, num_heads, vdim, head_dim, lam, out_scale, eps) -> None:
    """``out[t, h] = unit_rms(a1 - lam * a2) * out_scale * sigmoid(gate[t, h])`` over a head's
    ``vdim`` values, a1 / a2 the two maps' rows of ``attn`` [T, 2 H * head_dim]."""
    _check(heads().vx_diff_combine(
        _p(attn), _code(attn.dtype), attn.stride(0), _p(gate), 0 if gate is None else _pitched(gate, "gate"),
        _p(out), out.stride(0), num_tokens, num_heads, vdim, head_dim, float(lam), float(out_scale), float(eps),
        _stream()), "diff_combine")


def clamped_glu(gate_up, out, num_tokens, inner, limit, alpha, up_shift, cubic: float = 0.0) -> None:
    """``out = g * sigmoid(alpha * (g + cubic * g^3)) * (u + up_shift)`` with ``g = min(gate, limit)``, ``u =
    clamp(up, -limit, limit)`` (no clamps when ``limit`` is 0); gate columns first in ``gate_up``."""
    _check(heads().vx_clamped_glu(_p(gate_up), _code(gate_up.dtype), _pitched(gate_up, "gate_up"), _p(out),
                                  out.stride(0), num_tokens, inner, float(limit or 0.0), float(alpha),
                                  float(up_shift), float(cubic), _stream()), "clamped_glu")
