"""Generic batched GEMM with fused epilogue: the Python face of `csrc/gemm_tcgen05.cu`.

    D_z[r, n] = epilogue(alpha * sum_k A_z[r, k] * B_z[n, k]),      z = z_hi * zlo_n + z_lo

Operands are *views into flat storages* described by strides (in elements), so one kernel serves the 1x1
convolutions, the longitude DFTs, the per-order Legendre contractions and the per-degree complex spectral
contraction without any intermediate transposes.  On CUDA tensors the tcgen05 kernel runs; on CPU tensors a
bit-faithful emulation of the same addressing is used, so that the layout choreography of every caller
is testable without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _ext

ACT_NONE, ACT_GELU, ACT_DGELU, ACT_RELU, ACT_DRELU, ACT_SHRINK, ACT_DSHRINK = 0, 1, 2, 3, 4, 5, 6
ACT_MULAUX = 8      # multiply by the epilogue operand itself (a derivative saved by the forward pass: `preact_deriv`)
BIAS_NONE, BIAS_ROW, BIAS_COL = 0, 1, 2
_BIG = 1 << 30


@dataclass
class Operand:
    """A (rows x K) matrix batch inside `tensor`'s storage.

    mn_major=False: element (row, k) at offset + row*ld + k         (k contiguous)
    mn_major=True : element (row, k) at offset + k*ld + row         (row contiguous)
    plus z_lo*zs_lo + z_hi*zs_hi for the batch index.
    """

    tensor: torch.Tensor
    ld: int
    mn_major: bool = False
    offset: int = 0
    zs_lo: int = 0
    zs_hi: int = 0


@dataclass
class Output:
    """Destination addressing: offset + z_hi*d_zhi + z_lo*d_zlo + (r//rdiv)*rs_hi + (r%rdiv)*rs_lo + (n//ndiv)*ns_hi + n%ndiv."""

    tensor: torch.Tensor
    rs_lo: int
    offset: int = 0
    rdiv: int = _BIG
    rs_hi: int = 0
    ndiv: int = _BIG
    ns_hi: int = 0
    d_zlo: int = 0
    d_zhi: int = 0


@dataclass
class Tri:
    """Known-zero structure as affine functions of z_hi: valid rows [rmin, rmax), contributing k in [kmin, kmax)."""

    rmin_a: int = 0
    rmin_b: int = 0
    rmax_a: int = 0
    rmax_b: int = _BIG
    kmin_a: int = 0
    kmin_b: int = 0
    kmax_a: int = 0
    kmax_b: int = _BIG


@dataclass
class Segment:
    """One k-range of a B operand that is spread over several devices.

    `source` is the tensor holding the range on CPU (emulation) or the device address of the peer's buffer as an
    int on CUDA; all segments share the strides of the `Operand` they replace.  `length` is the k extent of the
    range, `a_pos` the k coordinate at which the matching columns of A start (a multiple of 64 elements so that
    TMA coordinates stay 16-byte aligned), `g_start` the global k index of the range for `Tri.kmin/kmax`.
    """

    source: object
    length: int
    a_pos: int
    g_start: int


def _flat(t: torch.Tensor) -> torch.Tensor:
    """1-D view over the whole storage extent used by `t` (t must be non-overlapping and dense or a slice)."""
    if t.is_contiguous():
        return t.view(-1)
    # generic: view the underlying storage from the tensor's storage offset onward
    n = t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()
    return t.as_strided((n,), (1,))


def _gelu_derivative(x: torch.Tensor) -> torch.Tensor:
    if _ext.gelu_approximation() == "tanh":
        u = 0.7978845608028654 * (x + 0.044715 * x ** 3)
        t = torch.tanh(u)
        return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * 0.7978845608028654 * (1.0 + 3 * 0.044715 * x * x)
    cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
    return cdf + x * pdf


def _emulate(M, N, K, A: Operand, B: Operand, D: Output, zlo_n, zhi_n, alpha, bias, bias_mode, act, resid, resid_offset,
             preact, preact_offset, accumulate, tri: Tri, segments=None, act_param: float = 0.0, bias_zs: int = 0,
             preact_deriv: bool = False):
    fa, fb, fd = _flat(A.tensor), _flat(B.tensor), _flat(D.tensor)
    cdt = torch.float64 if fa.dtype == torch.float64 else torch.float32

    def view(op: Operand, flat, rows, kext):
        rs, ks = (1, op.ld) if op.mn_major else (op.ld, 1)
        return flat[op.offset:].as_strided((zhi_n, zlo_n, rows, kext), (op.zs_hi, op.zs_lo, rs, ks)).to(cdt)

    a = view(A, fa, M, K)
    dev = fa.device
    if segments:
        # B gathered from several sources; columns of A outside every segment meet zeros (TMA out-of-bounds fill)
        b = torch.zeros(zhi_n, zlo_n, N, K, dtype=cdt, device=dev)
        k = torch.full((K,), -1, dtype=torch.long, device=dev)
        for sg in segments:
            b[..., sg.a_pos: sg.a_pos + sg.length] = view(B, _flat(sg.source), N, sg.length)
            k[sg.a_pos: sg.a_pos + sg.length] = torch.arange(sg.g_start, sg.g_start + sg.length, device=dev)
        k = k.view(1, 1, 1, -1)
    else:
        b = view(B, fb, N, K)
        k = torch.arange(K, device=dev).view(1, 1, 1, -1)
    zh = torch.arange(zhi_n, device=dev).view(-1, 1, 1, 1)
    r = torch.arange(M, device=dev).view(1, 1, -1, 1)
    kmask = (k >= tri.kmin_a * zh + tri.kmin_b) & (k < tri.kmax_a * zh + tri.kmax_b) & (k >= 0)
    a = a * kmask.to(cdt)
    acc = torch.matmul(a, b.transpose(-1, -2))  # [zh, zl, M, N]
    rmask = (r >= tri.rmin_a * zh + tri.rmin_b) & (r < tri.rmax_a * zh + tri.rmax_b)
    acc = acc * rmask.to(cdt)
    acc = acc * alpha
    if bias is not None and bias_zs:
        bz = bias.to(cdt).reshape(-1).as_strided((zlo_n, M if bias_mode == BIAS_ROW else N), (bias_zs, 1))
        acc = acc + (bz.view(1, zlo_n, -1, 1) if bias_mode == BIAS_ROW else bz.view(1, zlo_n, 1, -1))
    elif bias is not None and bias_mode == BIAS_ROW:
        acc = acc + bias.to(cdt).view(1, 1, -1, 1)[:, :, :M]
    elif bias is not None and bias_mode == BIAS_COL:
        acc = acc + bias.to(cdt).view(1, 1, 1, -1)[..., :N]
    zl = torch.arange(zlo_n, device=dev).view(1, -1, 1, 1)
    n = torch.arange(N, device=dev).view(1, 1, 1, -1)
    idx = (D.offset + zh * D.d_zhi + zl * D.d_zlo + (r // D.rdiv) * D.rs_hi + (r % D.rdiv) * D.rs_lo
           + (n // D.ndiv) * D.ns_hi + (n % D.ndiv))
    idx = idx.expand(zhi_n, zlo_n, M, N).reshape(-1)
    if preact is not None:
        second = _gelu_derivative(acc) if (preact_deriv and act == ACT_GELU) else acc
        _flat(preact).index_put_((idx - D.offset + preact_offset,), second.reshape(-1).to(preact.dtype))
    if act == ACT_GELU:
        acc = torch.nn.functional.gelu(acc, approximate=_ext.gelu_approximation())
    elif act == ACT_RELU:
        acc = torch.relu(acc)
    elif act == ACT_SHRINK:
        acc = torch.nn.functional.softshrink(acc, lambd=float(act_param))
    if resid is not None:
        rv = _flat(resid)[idx - D.offset + resid_offset].to(cdt).view_as(acc)
        if act == ACT_DRELU:
            acc = acc * (rv > 0).to(cdt)
        elif act == ACT_DSHRINK:
            acc = acc * (rv != 0).to(cdt)
        elif act == ACT_DGELU:
            acc = acc * _gelu_derivative(rv)
        elif act == ACT_MULAUX:
            acc = acc * rv
        else:
            acc = acc + rv
    vals = acc.reshape(-1).to(fd.dtype)
    if accumulate:
        fd.index_add_(0, idx, vals)
    else:
        fd.index_put_((idx,), vals)


def gemm(M: int, N: int, K: int, A: Operand, B: Operand, D: Output, *, zlo_n: int = 1, zhi_n: int = 1, alpha: float = 1.0,
         bias: Optional[torch.Tensor] = None, bias_mode: int = BIAS_NONE, act: int = ACT_NONE,
         resid: Optional[torch.Tensor] = None, resid_offset: int = 0, preact: Optional[torch.Tensor] = None,
         preact_offset: int = 0, accumulate: bool = False, splits: int = 1, tri: Optional[Tri] = None, bn: int = 0,
         segments=None, sync=None, dests=None, act_param: float = 0.0, bias_zs: int = 0,
         preact_deriv: bool = False) -> None:
    """Run the batched GEMM described above, writing into `D.tensor` in place.

    `segments` (list of `Segment`) spreads the k axis of B over several devices: `K` is then the padded k extent
    of A and `B.tensor` only supplies dtype and strides.  `sync` is the 31-entry handshake descriptor built by
    `makani_b200.parallel.peer.sync_descriptor` (CUDA only).  `dests` lists device addresses of additional copies of
    the output buffer (peers' memory) that receive the same bf16 stores as `D.tensor`.

    `preact` receives the value before the activation; with `preact_deriv` (act = ACT_GELU only) it receives GELU' of
    that value instead, which the backward pass multiplies in with `act=ACT_MULAUX, resid=<that tensor>`."""
    tri = tri or Tri()
    assert not preact_deriv or (act == ACT_GELU and preact is not None)
    if bias is None:
        bias_mode = BIAS_NONE
    if not A.tensor.is_cuda:
        _emulate(M, N, K, A, B, D, zlo_n, zhi_n, alpha, bias, bias_mode, act, resid, resid_offset, preact, preact_offset,
                 accumulate, tri, segments, act_param, bias_zs, preact_deriv)
        return
    ext = _ext.require()
    ip = [M, N, K, zlo_n, zhi_n, splits, bn,
          tri.rmin_a, tri.rmin_b, tri.rmax_a, tri.rmax_b, tri.kmin_a, tri.kmin_b, tri.kmax_a, tri.kmax_b,
          A.offset, int(A.mn_major), A.ld, A.zs_lo, A.zs_hi,
          B.offset, int(B.mn_major), B.ld, B.zs_lo, B.zs_hi,
          D.offset, int(accumulate), D.d_zlo, D.d_zhi, D.rdiv, D.rs_hi, D.rs_lo, D.ndiv, D.ns_hi,
          bias_mode, act | (256 if preact_deriv else 0), resid_offset, preact_offset, _f32_bits(act_param), int(bias_zs)]
    if segments or sync or dests:
        seg = []
        if segments and len(segments) > 1:
            seg = [len(segments)]
            for sg in segments:
                assert sg.a_pos % 64 == 0, "segment start in A must be a multiple of 64 elements"
                seg += [int(sg.source), int(sg.length), int(sg.a_pos), int(sg.g_start)]
        elif segments:
            raise ValueError("a single-segment operand is an ordinary operand: pass it as B")
        ext.gemm_peer(A.tensor, B.tensor, D.tensor, bias, resid, preact, ip, float(alpha), seg, list(sync or []),
                      [int(d) for d in (dests or [])])
        return
    ext.gemm(A.tensor, B.tensor, D.tensor, bias, resid, preact, ip, float(alpha))


def _f32_bits(x: float) -> int:
    import struct
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m
