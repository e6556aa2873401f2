"""torch.Tensor-level wrappers around the C-ABI entry points (device pointers in, nothing
allocated by the library).  These are the only functions that touch ctypes."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_DTYPE_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
DEQ_FUSED, DEQ_PYTORCH, DEQ_TRITON = 0, 1, 2


def _stream(t: torch.Tensor) -> int:
    _lib.init_device(t.device.index if t.device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(t.device).cuda_stream


class DeviceTimeout(RuntimeError):
    """A bounded device-side wait gave up (``LLNV_E_TIMEOUT``): results of the affected step are invalid."""


def check_status(device=None) -> None:
    """Synchronise the current stream of ``device`` and raise ``DeviceTimeout`` if a kernel's bounded wait
    (an mbarrier wait, a peer barrier) gave up since the last check (``llnv_check_status``; clears the flag)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        rc = _lib.lib().llnv_check_status(torch.cuda.current_stream(dev).cuda_stream)
    if rc == -3:
        raise DeviceTimeout(_lib.lib().llnv_last_error().decode("utf-8", "replace"))
    _check(rc)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor (the NVFP4 path has no CPU implementation)")


def _check(rc: int) -> None:
    if rc != 0:
        msg = _lib.lib().llnv_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"llnvfp4 error {rc}: {msg}")


def padded_rows(m: int) -> int:
    return (m + 127) // 128 * 128


def amax_bf16(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _require_cuda(x, "x")
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        out = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_amax_bf16(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), out.data_ptr(), _stream(x)))
    return out


def _group_args(group):
    """(slot pointer table, signal pointer table, rank, world, epoch pointer) of a peer arena (``sp.PeerArena``)."""
    return (_ptr_table([b + group.SIGNAL_BYTES for b in group.base]), _ptr_table(group.base), group.rank, group.world,
            group.epoch.data_ptr())


def quantize_nvfp4(x: torch.Tensor, rule_id: int, amax: torch.Tensor | None = None, codes=None, sf=None,
                   amax_given: bool | None = None, group=None):
    """bf16 [M, K] (K % 64 == 0, unit column stride) -> (codes [Mp, K/2] u8, sf [Mp*K/16] e4m3, amax [1] f32).

    A contiguous 3-D ``x`` [shards, M, K / shards] is read as the column-sharded form of the [M, K]
    matrix (``llnv_quantize_nvfp4_ex``).

    ``amax`` is the fp32 tensor-scale buffer.  With ``amax_given`` (default: true when a buffer is
    passed) it is read as the scale; otherwise it is computed on the device into that buffer (or a
    new one).  ``codes`` / ``sf`` may be preallocated slot buffers (KV cache) written in place.
    ``group`` (a ``sp.PeerArena``): ``amax`` holds this rank's amax of its shard; the quantize kernel MAX-reduces it over
    the group before its first block and leaves the group maximum in ``amax`` (``llnv_quantize_nvfp4_group``).
    """
    _require_cuda(x, "x")
    shards = 1
    if x.dim() == 3 and x.dtype == torch.bfloat16 and x.is_contiguous():
        shards, m, ks = x.shape
        k, ldx = shards * ks, ks
    elif x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("quantize_nvfp4 expects a 2-D bfloat16 or float16 tensor (or a contiguous bfloat16 [shards, M, K/shards] one)")
    else:
        if x.stride(1) != 1:
            x = x.contiguous()
        m, k = x.shape
        ldx = x.stride(0)
    mp = padded_rows(m)
    if codes is None:
        codes = torch.empty((mp, k // 2), dtype=torch.uint8, device=x.device)
    if sf is None:
        sf = torch.empty(mp * k // 16, dtype=torch.float8_e4m3fn, device=x.device)
    given = (amax is not None) if amax_given is None else bool(amax_given)
    if amax is None:
        if given:
            raise ValueError("amax_given needs an amax tensor")
        amax = torch.empty(1, dtype=torch.float32, device=x.device)
    if x.dtype == torch.float16:
        if group is not None:
            raise ValueError("the group form takes bfloat16 input")
        with torch.cuda.device(x.device):
            _check(_lib.lib().llnv_quantize_nvfp4_f16(x.data_ptr(), m, k, ldx, rule_id, codes.data_ptr(), sf.data_ptr(),
                                                      amax.data_ptr(), 1 if given else 0, _stream(x)))
        return codes, sf, amax
    with torch.cuda.device(x.device):
        if group is not None:
            if not given:
                raise ValueError("the group form needs this rank's amax in `amax`")
            _check(_lib.lib().llnv_quantize_nvfp4_group(x.data_ptr(), m, k, ldx, rule_id, codes.data_ptr(), sf.data_ptr(),
                                                        amax.data_ptr(), shards, *_group_args(group), _stream(x)))
        else:
            _check(_lib.lib().llnv_quantize_nvfp4_ex(x.data_ptr(), m, k, ldx, rule_id, codes.data_ptr(), sf.data_ptr(),
                                                     amax.data_ptr(), 1 if given else 0, shards, _stream(x)))
    return codes, sf, amax


def _quant_outputs(x, m, c, codes, sf, amax):
    mp = padded_rows(m)
    if codes is None:
        codes = torch.empty((mp, c // 2), dtype=torch.uint8, device=x.device)
    if sf is None:
        sf = torch.empty(mp * c // 16, dtype=torch.float8_e4m3fn, device=x.device)
    if amax is None:
        amax = torch.empty(1, dtype=torch.float32, device=x.device)
    return codes, sf, amax


def adaln_quantize_nvfp4(x, scale, shift, frame_rows, rule_id, eps=1e-6, add_one=True, *, want_y=False, codes=None,
                         sf=None, amax=None, row_stats=None, row_offset=0, phase=0, y_only=False, group=None):
    """LayerNorm(no affine) -> (1 + scale[f]) * x + shift[f] (bf16 rounding points of the reference)
    fused with the NVFP4 quantize of the result.  x: bf16 [M, C]; scale/shift: bf16 [F, C] views
    (row stride free).  Returns (codes, sf, amax, y or None); with ``y_only`` nothing is quantized
    (codes and sf are None) and only y is produced.  ``group`` (a ``sp.PeerArena``): the tensor amax is MAX-reduced
    over the group inside the quantize kernel (``llnv_adaln_quantize_nvfp4_group``)."""
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise RuntimeError("adaln_quantize_nvfp4 expects a 2-D bfloat16 tensor with unit column stride")
    if scale.dim() != 2 or shift.dim() != 2 or scale.stride(1) != 1 or shift.stride(1) != 1 or scale.stride(0) != shift.stride(0):
        raise RuntimeError("scale and shift must be [frames, C] views with the same row stride")
    m, c = x.shape
    if y_only:
        want_y, codes, sf = True, None, None
        amax = amax if amax is not None else torch.empty(1, dtype=torch.float32, device=x.device)
    else:
        codes, sf, amax = _quant_outputs(x, m, c, codes, sf, amax)
    if row_stats is None:
        row_stats = torch.empty(2 * max(m, 1), dtype=torch.float32, device=x.device)
    y = torch.empty((m, c), dtype=torch.bfloat16, device=x.device) if want_y else None
    if group is not None:
        if want_y or phase != 0:
            raise ValueError("the group form runs both passes and produces no y")
        with torch.cuda.device(x.device):
            _check(_lib.lib().llnv_adaln_quantize_nvfp4_group(
                x.data_ptr(), m, c, x.stride(0), scale.data_ptr(), shift.data_ptr(), scale.stride(0), int(frame_rows), float(eps),
                1 if add_one else 0, rule_id, codes.data_ptr(), sf.data_ptr(), amax.data_ptr(), row_stats.data_ptr(), int(row_offset),
                *_group_args(group), _stream(x)))
        return codes, sf, amax, None
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_adaln_quantize_nvfp4_ex(
            x.data_ptr(), m, c, x.stride(0), scale.data_ptr(), shift.data_ptr(), scale.stride(0), int(frame_rows), float(eps),
            1 if add_one else 0, rule_id, codes.data_ptr() if codes is not None else None,
            sf.data_ptr() if sf is not None else None, amax.data_ptr(),
            y.data_ptr() if y is not None else None, c, row_stats.data_ptr(), int(row_offset), int(phase), _stream(x)))
    return codes, sf, amax, y


def layernorm_quantize_nvfp4(x, weight, bias, rule_id, eps=1e-6, *, want_y=False, codes=None, sf=None, amax=None,
                             row_stats=None, phase=0, group=None):
    """Affine LayerNorm fused with the NVFP4 quantize of its output.  Returns (codes, sf, amax, y or None).
    ``group`` (a ``sp.PeerArena``): the tensor amax is MAX-reduced over the group inside the quantize kernel."""
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise RuntimeError("layernorm_quantize_nvfp4 expects a 2-D bfloat16 tensor with unit column stride")
    m, c = x.shape
    codes, sf, amax = _quant_outputs(x, m, c, codes, sf, amax)
    if row_stats is None:
        row_stats = torch.empty(2 * max(m, 1), dtype=torch.float32, device=x.device)
    y = torch.empty((m, c), dtype=torch.bfloat16, device=x.device) if want_y else None
    if group is not None:
        if want_y or phase != 0:
            raise ValueError("the group form runs both passes and produces no y")
        with torch.cuda.device(x.device):
            _check(_lib.lib().llnv_layernorm_quantize_nvfp4_group(
                x.data_ptr(), m, c, x.stride(0), weight.data_ptr(), bias.data_ptr(), float(eps), rule_id, codes.data_ptr(),
                sf.data_ptr(), amax.data_ptr(), row_stats.data_ptr(), *_group_args(group), _stream(x)))
        return codes, sf, amax, None
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_layernorm_quantize_nvfp4_ex(
            x.data_ptr(), m, c, x.stride(0), weight.data_ptr(), bias.data_ptr(), float(eps), rule_id, codes.data_ptr(),
            sf.data_ptr(), amax.data_ptr(), y.data_ptr() if y is not None else None, c, row_stats.data_ptr(), int(phase),
            _stream(x)))
    return codes, sf, amax, y


def rmsnorm_rope(x, weight=None, cos=None, sin=None, eps=1e-6, *, out=None, out_smooth=None, want_smooth=False,
                 amax_out=None, want_amax=False, shards=1):
    """RMSNorm (if ``weight``) -> per-head RoPE (if ``cos``/``sin``, fp32 [S, 64]) on bf16 [S, C];
    optionally the k_smooth copy and max|out|.  Returns (out, out_smooth or None, amax or None).
    With ``shards`` > 1 the outputs are contiguous [shards, S, C / shards] tensors (head-sharded)."""
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise RuntimeError("rmsnorm_rope expects a 2-D bfloat16 tensor with unit column stride")
    s, c = x.shape
    oshape = (s, c) if shards == 1 else (shards, s, c // shards)
    if out is None:
        out = torch.empty(oshape, dtype=torch.bfloat16, device=x.device)
    if out_smooth is None and want_smooth:
        out_smooth = torch.empty(oshape, dtype=torch.bfloat16, device=x.device)
    if shards > 1:
        for t in (out, out_smooth):
            if t is not None and (tuple(t.shape) != oshape or not t.is_contiguous()):
                raise RuntimeError("sharded outputs must be contiguous [shards, S, C / shards]")
    if amax_out is None and want_amax:
        amax_out = torch.empty(1, dtype=torch.float32, device=x.device)
    if cos is not None and (cos.dtype != torch.float32 or cos.shape != (s, 64) or not cos.is_contiguous() or not sin.is_contiguous()):
        raise RuntimeError("cos/sin must be contiguous float32 [S, 64]")
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_rmsnorm_rope_ex(
            x.data_ptr(), s, c, x.stride(0), weight.data_ptr() if weight is not None else None, float(eps),
            cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
            out.data_ptr(), out.stride(-2), out_smooth.data_ptr() if out_smooth is not None else None,
            out_smooth.stride(-2) if out_smooth is not None else 0,
            amax_out.data_ptr() if amax_out is not None else None, shards, _stream(x)))
    return out, out_smooth, amax_out


def quantize_nvfp4_pair(x0, x1, rule_id, q0, q1, amax_given=True):
    """Quantize two bf16 [M, K] tensors of the same shape in one launch into the preallocated
    QuantizedTensor-like targets q0 / q1 (``values``, ``scale_factors``, ``amax``)."""
    _require_cuda(x0, "x0")
    if x0.shape != x1.shape or x0.stride(0) != x1.stride(0) or x0.stride(1) != 1 or x1.stride(1) != 1 or x0.dtype != torch.bfloat16:
        raise RuntimeError("quantize_nvfp4_pair expects two bfloat16 [M, K] tensors of the same shape and row stride")
    m, k = x0.shape
    with torch.cuda.device(x0.device):
        _check(_lib.lib().llnv_quantize_nvfp4_pair(x0.data_ptr(), x1.data_ptr(), m, k, x0.stride(0), rule_id, q0.values.data_ptr(),
                                                   q0.scale_factors.data_ptr(), q0.amax.data_ptr(), q1.values.data_ptr(),
                                                   q1.scale_factors.data_ptr(), q1.amax.data_ptr(), 1 if amax_given else 0, _stream(x0)))


def _ptr_table(ptrs):
    arr = (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr


def rmsnorm_rope_scatter(x, weight, cos, sin, eps, out_ptrs, ldo, smooth_ptrs=None, lds=0, amax_out=None):
    """``rmsnorm_rope`` whose head shard r is stored at ``out_ptrs[r]`` (and ``smooth_ptrs[r]``): raw
    device addresses, possibly on other GPUs of the node.  See ``llnv_rmsnorm_rope_scatter``."""
    _require_cuda(x, "x")
    s, c = x.shape
    shards = len(out_ptrs)
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_rmsnorm_rope_scatter(
            x.data_ptr(), s, c, x.stride(0), weight.data_ptr() if weight is not None else None, float(eps),
            cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None,
            _ptr_table(out_ptrs), ldo, _ptr_table(smooth_ptrs) if smooth_ptrs is not None else None, lds,
            amax_out.data_ptr() if amax_out is not None else None, shards, _stream(x)))


def rmsnorm_rope_qk(xq, wq, q_ptrs, ldq, xk, wk, k_ptrs, ldk, k_smooth_ptrs, lds, k_amax, cos, sin, eps):
    """The q and the k prologue of a block in one launch (``llnv_rmsnorm_rope_qk``); outputs are raw
    device addresses, one per head shard."""
    _require_cuda(xq, "xq")
    s, c = xq.shape
    with torch.cuda.device(xq.device):
        _check(_lib.lib().llnv_rmsnorm_rope_qk(
            xq.data_ptr(), xq.stride(0), wq.data_ptr(), _ptr_table(q_ptrs), ldq, xk.data_ptr(), xk.stride(0), wk.data_ptr(),
            _ptr_table(k_ptrs), ldk, _ptr_table(k_smooth_ptrs) if k_smooth_ptrs is not None else None, lds,
            k_amax.data_ptr() if k_amax is not None else None, s, c, float(eps), cos.data_ptr(), sin.data_ptr(), len(q_ptrs), _stream(xq)))


def scatter_2d(src, src_shard_bytes, dst_ptrs, dst_pitch, rows, row_bytes):
    """Push ``rows`` x ``row_bytes`` blocks of the 2-D tensor ``src`` (block r starts r * src_shard_bytes
    bytes in) to the raw device addresses ``dst_ptrs`` (possibly peer memory).  See ``llnv_scatter_2d``."""
    _require_cuda(src, "src")
    with torch.cuda.device(src.device):
        _check(_lib.lib().llnv_scatter_2d(src.data_ptr(), src_shard_bytes, src.stride(0) * src.element_size(), _ptr_table(dst_ptrs),
                                          dst_pitch, rows, row_bytes, len(dst_ptrs), _stream(src)))


_LINEAR_ACT = {None: 0, "none": 0, "gelu_tanh": 1, "silu": 2}


def linear_bf16(x, w, bias=None, act=None, out=None):
    """``act(x @ w.T + bias)`` for bf16 ``x`` [M, K], ``w`` [N, K], ``bias`` [N] on the tcgen05 bf16 kernel
    (``llnv_linear_bf16``): the Linear of the layers the reference keeps in bf16.  ``act``: None,
    "gelu_tanh" or "silu".  Unit column strides; K, N and the row strides multiples of 8."""
    _require_cuda(x, "x")
    if act not in _LINEAR_ACT:
        raise ValueError(f"act must be one of {sorted(k for k in _LINEAR_ACT if k)} or None")
    for name, t in (("x", x), ("w", w)):
        if t.dim() != 2 or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise RuntimeError(f"{name} must be a 2-D bfloat16 tensor with unit column stride")
    if x.shape[1] != w.shape[1]:
        raise RuntimeError(f"x is [M, {x.shape[1]}] but w is [N, {w.shape[1]}]")
    m, k = x.shape
    n = w.shape[0]
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != n or not bias.is_contiguous()):
        raise RuntimeError("bias must be a contiguous bfloat16 tensor of N values")
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    elif out.shape != (m, n) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise RuntimeError("out must be bfloat16 [M, N] with unit column stride")
    with torch.cuda.device(x.device):
        _check(_lib.lib().llnv_linear_bf16(x.data_ptr(), x.stride(0) if m > 1 else max(k, x.stride(0)), w.data_ptr(), w.stride(0),
                                           None if bias is None else bias.data_ptr(), _LINEAR_ACT[act], m, n, k, out.data_ptr(),
                                           out.stride(0) if m > 1 else max(n, out.stride(0)), _stream(x)))
    return out


def _latent_view(latent, channels_first):
    if latent.dim() != 4 or latent.dtype != torch.bfloat16 or latent.stride(3) != 1 or latent.stride(2) != latent.shape[3]:
        raise RuntimeError("latent must be a 4-D bfloat16 tensor whose two image axes are contiguous")
    if latent.shape[2] % 2 or latent.shape[3] % 2:
        raise RuntimeError("latent height and width must be even (patch 1 x 2 x 2)")
    c_ax, f_ax = (0, 1) if channels_first else (1, 0)
    return latent.shape[c_ax], latent.shape[f_ax], latent.stride(c_ax), latent.stride(f_ax), latent.shape[2] // 2, latent.shape[3] // 2


def patchify(latent, channels_first=True, out=None):
    """bf16 latent [C, F, H, W] (or [F, C, H, W] with ``channels_first=False``) -> tokens [F*H/2*W/2, 4*C],
    features ordered (c, kh, kw): the input of the patch embedding (``llnv_patchify``)."""
    _require_cuda(latent, "latent")
    C, F, sc, sf, h, w = _latent_view(latent, channels_first)
    if out is None:
        out = torch.empty((F * h * w, 4 * C), dtype=torch.bfloat16, device=latent.device)
    elif out.shape != (F * h * w, 4 * C) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise RuntimeError("out must be bfloat16 [F*h*w, 4*C] with unit column stride")
    with torch.cuda.device(latent.device):
        _check(_lib.lib().llnv_patchify(latent.data_ptr(), sc, sf, out.data_ptr(), out.stride(0), C, F, h, w, _stream(latent)))
    return out


def unpatchify(tokens, out, channels_first=True):
    """Tokens [F*h*w, 4*C] (features (c, kh, kw)) -> the bf16 latent ``out`` [C, F, 2h, 2w] (or [F, C, 2h, 2w]);
    the inverse of ``patchify`` (``llnv_unpatchify``)."""
    _require_cuda(tokens, "tokens")
    C, F, sc, sf, h, w = _latent_view(out, channels_first)
    if tokens.shape != (F * h * w, 4 * C) or tokens.dtype != torch.bfloat16 or tokens.stride(1) != 1 or tokens.device != out.device:
        raise RuntimeError("tokens must be bfloat16 [F*h*w, 4*C] with unit column stride on the device of out")
    with torch.cuda.device(tokens.device):
        _check(_lib.lib().llnv_unpatchify(tokens.data_ptr(), tokens.stride(0), out.data_ptr(), sc, sf, C, F, h, w, _stream(tokens)))
    return out


def peer_barrier(signal_ptrs, rank, epoch):
    """Stream-ordered barrier over the GPUs whose signal areas are ``signal_ptrs`` (``llnv_peer_barrier``)."""
    with torch.cuda.device(epoch.device):
        _check(_lib.lib().llnv_peer_barrier(_ptr_table(signal_ptrs), rank, len(signal_ptrs), epoch.data_ptr(), _stream(epoch)))


def peer_allreduce_max(vals, slot_ptrs, signal_ptrs, rank, epoch):
    """In-place MAX all-reduce of a small fp32 tensor over the GPUs of a peer arena (``llnv_peer_allreduce_max``)."""
    with torch.cuda.device(vals.device):
        _check(_lib.lib().llnv_peer_allreduce_max(vals.data_ptr(), vals.numel(), _ptr_table(slot_ptrs), _ptr_table(signal_ptrs), rank,
                                                  len(signal_ptrs), epoch.data_ptr(), _stream(vals)))


SPLIT_TAIL = -1          # LLNV_ATTN_SPLIT_TAIL: cut the tiles of the last partial wave once (see include/llnvfp4.h)


def _attention_workspace(lib, lq, heads, key_splits, workspace, device):
    """(tensor, bytes) of the partial-result workspace a split or tail-balanced call needs: the caller's ``workspace``
    (uint8, at least llnv_attention_workspace_bytes) or a fresh allocation."""
    if not (key_splits > 1 or key_splits == SPLIT_TAIL):
        return None, 0
    ws_bytes = lib.llnv_attention_workspace_bytes(lq, heads, key_splits)
    if workspace is not None:
        if workspace.dtype != torch.uint8 or not workspace.is_contiguous() or workspace.numel() < ws_bytes or workspace.device != device:
            raise RuntimeError(f"attention workspace must be a contiguous uint8 tensor of at least {ws_bytes} bytes on the device of q")
        return workspace, workspace.numel()
    return torch.empty(ws_bytes, dtype=torch.uint8, device=device), ws_bytes


def attention_workspace_bytes(lq, lk, heads, key_splits=None):
    """Bytes of workspace ``attention_bf16`` / ``attention_nvfp4kv`` use for this shape (0 when the call is not split);
    ``key_splits`` None = what the library proposes for the current device."""
    lib = _lib.lib()
    if key_splits is None:
        key_splits = lib.llnv_attention_key_splits(lq, lk, heads)
    return int(lib.llnv_attention_workspace_bytes(lq, heads, key_splits)) if (key_splits > 1 or key_splits == SPLIT_TAIL) else 0


def attention_bf16(q, k, v, heads, scale=None, out=None, key_splits=None, out_amax=None, workspace=None):
    """softmax(q k^T * scale) v per head, non-causal.  q: bf16 [Lq, heads*128]; k, v: bf16 [Lk, heads*128]
    (row strides free, unit column stride).  Returns bf16 [Lq, heads*128].  ``key_splits`` > 1 splits
    the key window over several CTAs per query tile (default: what the library proposes for the
    device, 1 unless the tiles alone leave most SMs idle).  ``out_amax`` (fp32 [1]) receives max |out|.
    ``workspace``: a uint8 tensor for the partial results of a split call (``attention_workspace_bytes``); allocated
    per call when omitted."""
    _require_cuda(q, "q")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dim() != 2 or t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != heads * 128:
            raise RuntimeError(f"{name} must be bfloat16 [tokens, heads*128] with unit column stride")
    if k.shape[0] != v.shape[0]:
        raise RuntimeError("k and v must have the same number of tokens")
    if out is None:
        out = torch.empty((q.shape[0], heads * 128), dtype=torch.bfloat16, device=q.device)
    if scale is None:
        scale = 128 ** -0.5
    lib = _lib.lib()
    with torch.cuda.device(q.device):
        if key_splits is None:
            key_splits = lib.llnv_attention_key_splits(q.shape[0], k.shape[0], heads)
        ws, ws_bytes = _attention_workspace(lib, q.shape[0], heads, key_splits, workspace, q.device)
        _check(lib.llnv_attention_bf16_ex(q.data_ptr(), q.shape[0], q.stride(0), k.data_ptr(), v.data_ptr(), k.shape[0],
                                          k.stride(0), v.stride(0), heads, float(scale), out.data_ptr(), out.stride(0),
                                          int(key_splits), ws.data_ptr() if ws is not None else None, ws_bytes,
                                          out_amax.data_ptr() if out_amax is not None else None, _stream(q)))
    return out


def attention_nvfp4kv(q, k_blocks, v_blocks, block_tokens, k_cur, v_cur, heads, scale=None, out=None, key_splits=None,
                      out_amax=None, e2m1_max=6.0, e4m3_max=256.0, workspace=None):
    """Chunk attention over [cached NVFP4 blocks ... | current chunk (bf16)] without dequantizing the cache to
    memory (``llnv_attention_nvfp4kv``).  ``k_blocks`` / ``v_blocks``: cache blocks oldest first, each with
    ``values`` (uint8 [rows_padded, 64]), ``scale_factors`` and ``amax`` (a ``QuantizedTensor`` of
    ``block_tokens * heads`` rows of 128 channels, token-major / head-minor).  ``k_cur`` / ``v_cur``: bf16
    [L_cur, heads*128] (or None when the window is the cache alone).  Result: bf16 [Lq, heads*128], equal bit
    for bit to dequantizing the blocks into a window and calling ``attention_bf16`` on it."""
    _require_cuda(q, "q")
    if q.dim() != 2 or q.dtype != torch.bfloat16 or q.stride(1) != 1 or q.shape[1] != heads * 128:
        raise RuntimeError("q must be bfloat16 [tokens, heads*128] with unit column stride")
    n = len(k_blocks)
    if len(v_blocks) != n:
        raise RuntimeError("k_blocks and v_blocks must have the same length")
    for b in list(k_blocks) + list(v_blocks):
        v = b.values
        if v.dtype != torch.uint8 or v.dim() != 2 or v.shape[1] != 64 or not v.is_contiguous() or v.shape[0] < block_tokens * heads:
            raise RuntimeError("a cache block must be contiguous uint8 [rows_padded, 64] covering block_tokens * heads rows")
        if v.device != q.device or b.scale_factors.device != q.device or b.amax.device != q.device or b.amax.dtype != torch.float32:
            raise RuntimeError("cache blocks must live on the device of q, with float32 amax")
    l_cur = 0
    if k_cur is not None:
        for name, t in (("k_cur", k_cur), ("v_cur", v_cur)):
            if t is None or t.dim() != 2 or t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != heads * 128:
                raise RuntimeError(f"{name} must be bfloat16 [tokens, heads*128] with unit column stride")
        if k_cur.shape[0] != v_cur.shape[0]:
            raise RuntimeError("k_cur and v_cur must have the same number of tokens")
        l_cur = k_cur.shape[0]
    lk = n * block_tokens + l_cur
    if out is None:
        out = torch.empty((q.shape[0], heads * 128), dtype=torch.bfloat16, device=q.device)
    if scale is None:
        scale = 128 ** -0.5
    lib = _lib.lib()
    tab = lambda blocks, f: _ptr_table([f(b).data_ptr() for b in blocks]) if n else None
    with torch.cuda.device(q.device):
        if key_splits is None:
            key_splits = lib.llnv_attention_key_splits(q.shape[0], lk, heads)
        ws, ws_bytes = _attention_workspace(lib, q.shape[0], heads, key_splits, workspace, q.device)
        _check(lib.llnv_attention_nvfp4kv(
            q.data_ptr(), q.shape[0], q.stride(0),
            tab(k_blocks, lambda b: b.values), tab(k_blocks, lambda b: b.scale_factors), tab(k_blocks, lambda b: b.amax),
            tab(v_blocks, lambda b: b.values), tab(v_blocks, lambda b: b.scale_factors), tab(v_blocks, lambda b: b.amax),
            n, int(block_tokens), float(e2m1_max), float(e4m3_max),
            k_cur.data_ptr() if l_cur else None, v_cur.data_ptr() if l_cur else None, l_cur,
            k_cur.stride(0) if l_cur else 0, v_cur.stride(0) if l_cur else 0, heads, float(scale), out.data_ptr(), out.stride(0),
            int(key_splits), ws.data_ptr() if ws is not None else None, ws_bytes,
            out_amax.data_ptr() if out_amax is not None else None, _stream(q)))
    return out


def dequantize_nvfp4(codes, sf, amax, rows, cols, cols_padded, dtype, e2m1_max, e4m3_max, rounding=DEQ_PYTORCH):
    _require_cuda(codes, "codes")
    out = torch.empty((rows, cols), dtype=dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        _check(_lib.lib().llnv_dequantize_nvfp4(codes.data_ptr(), sf.data_ptr(), amax.data_ptr(), rows, cols, cols_padded,
                                                _DTYPE_CODES[dtype], float(e2m1_max), float(e4m3_max), rounding,
                                                out.data_ptr(), out.stride(0), _stream(codes)))
    return out


def kv_dequant(values, scale_factors, amax, num_heads, block_token_size, dtype, e2m1_max, e4m3_max,
               rounding=DEQ_FUSED, out=None):
    n = len(values)
    if n == 0:
        raise RuntimeError("values must contain at least one cache block")
    if not (len(scale_factors) == n and len(amax) == n):
        raise RuntimeError("values, scale_factors and amax must have the same length")
    _require_cuda(values[0], "values")
    dev = values[0].device
    if dtype not in _DTYPE_CODES:
        raise ValueError(f"Unsupported fused KV dequant dtype: {dtype}")
    for v, s, a in zip(values, scale_factors, amax):
        if v.dtype != torch.uint8 or v.dim() != 2 or v.shape[1] != 64:
            raise RuntimeError("KV dequant expects uint8 values of shape [rows_padded, 64] (head_dim 128)")
        if v.shape[0] < num_heads * block_token_size or v.shape[0] % 128 != 0:
            raise RuntimeError("values rows must be padded to a multiple of 128 and cover the block")
        if a.dtype != torch.float32:
            raise RuntimeError("amax tensors must be float32")
        if v.device != dev or s.device != dev or a.device != dev:
            raise RuntimeError("all KV block tensors must be on the same device")
        if not (v.is_contiguous() and s.is_contiguous() and a.is_contiguous()):
            raise RuntimeError("KV block tensors must be contiguous")
    if out is None:
        out = torch.empty((1, n * block_token_size, num_heads, 128), dtype=dtype, device=dev)
    arr = C.c_void_p * n
    cp = arr(*[v.data_ptr() for v in values])
    sp = arr(*[s.data_ptr() for s in scale_factors])
    ap = arr(*[a.data_ptr() for a in amax])
    with torch.cuda.device(dev):
        _check(_lib.lib().llnv_kv_dequant(cp, sp, ap, n, num_heads, block_token_size, _DTYPE_CODES[dtype],
                                          float(e2m1_max), float(e4m3_max), rounding, out.data_ptr(), _stream(values[0])))
    return out


def gemm_nvfp4(a_codes, a_sf, a_amax, a_rule, b_codes, b_sf, b_amax, b_rule, m, n, k, *, out=None, alpha=None,
               bias=None, act=0, residual=None, gate=None, frame_rows=0, out_amax=None, row_offset=0, tile=0,
               requant=None, requant_amax=None, store_out=True):
    """``epilogue(alpha * A @ B^T)`` -> bf16 [m, n]; see ``llnv_gemm_nvfp4`` in include/llnvfp4.h.
    ``tile``: 0 = tiling chosen by shape, 128 / 192 / 256 = that tile width, 2 = CTA-pair kernel.
    ``requant`` = (codes, sf) buffers: the epilogue also writes the NVFP4 form of the result (4-over-6 MSE rule)
    under the tensor amax ``requant_amax`` (fp32 [1], known before the call); with ``store_out=False`` the bf16
    result itself is not written and None is returned."""
    _require_cuda(a_codes, "a_codes")
    dev = a_codes.device
    if requant is None and not store_out:
        raise ValueError("store_out=False needs requant buffers")
    if out is None and store_out:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    epi = _lib.Epilogue()
    epi.alpha = alpha.data_ptr() if alpha is not None else None
    epi.bias = bias.data_ptr() if bias is not None else None
    epi.act = int(act)
    if residual is not None:
        epi.residual = residual.data_ptr()
        epi.ldr = residual.stride(0)
    if gate is not None:
        epi.gate = gate.data_ptr()
        epi.gate_stride = gate.stride(0)
        epi.frame_rows = int(frame_rows)
        epi.row_offset = int(row_offset)
    epi.out_amax = out_amax.data_ptr() if out_amax is not None else None
    if requant is not None:
        q_codes, q_sf = requant
        if requant_amax is None or requant_amax.dtype != torch.float32:
            raise ValueError("requant needs requant_amax (fp32 [1]): the tensor amax must be known before the GEMM runs")
        if q_codes.dtype != torch.uint8 or q_codes.numel() < padded_rows(m) * n // 2 or q_sf.numel() < padded_rows(m) * n // 16:
            raise RuntimeError("requant buffers must hold uint8 [Mp, N/2] codes and Mp*N/16 scale bytes")
        epi.q_codes, epi.q_sf, epi.q_amax, epi.q_rule = q_codes.data_ptr(), q_sf.data_ptr(), requant_amax.data_ptr(), 3
    with torch.cuda.device(dev):
        _check(_lib.lib().llnv_gemm_nvfp4_ex(a_codes.data_ptr(), a_sf.data_ptr(),
                                             a_amax.data_ptr() if a_amax is not None else None, a_rule,
                                             b_codes.data_ptr(), b_sf.data_ptr(),
                                             b_amax.data_ptr() if b_amax is not None else None, b_rule,
                                             m, n, k, C.byref(epi), out.data_ptr() if store_out else None,
                                             out.stride(0) if store_out else n, int(tile), _stream(a_codes)))
    return out if store_out else None


def gemm_nvfp4_grouped(a_codes, a_sf, a_amax, a_rule, b_codes, b_sf, b_amax, b_rule, m, n_each, k, outs, *, bias=None, act=0,
                       out_amax=None):
    """Two or three Linears sharing their input in one launch (``llnv_gemm_nvfp4_grouped``): ``b_codes`` /
    ``b_sf`` are the weights concatenated along N, ``b_amax`` an fp32 tensor with one amax per weight,
    ``outs`` the output tensors (bf16 [m, n_each], any row stride), ``out_amax`` a list of fp32 [1]
    tensors or None per output."""
    _require_cuda(a_codes, "a_codes")
    g = len(outs)
    epi = _lib.Epilogue()
    epi.bias = bias.data_ptr() if bias is not None else None
    epi.act = int(act)
    d = _ptr_table([o.data_ptr() for o in outs])
    ldd = (C.c_int64 * g)(*[o.stride(0) for o in outs])
    am = _ptr_table([(t.data_ptr() if t is not None else 0) for t in out_amax]) if out_amax is not None else None
    with torch.cuda.device(a_codes.device):
        _check(_lib.lib().llnv_gemm_nvfp4_grouped(a_codes.data_ptr(), a_sf.data_ptr(), a_amax.data_ptr(), a_rule, b_codes.data_ptr(),
                                                  b_sf.data_ptr(), b_amax.data_ptr(), b_rule, m, n_each, k, g, C.byref(epi), d, ldd, am,
                                                  _stream(a_codes)))
    return outs
