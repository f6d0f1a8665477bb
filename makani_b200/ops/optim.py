"""Fused multi-tensor Adam / AdamW: one kernel launch updates every parameter, its two moments and
(optionally) a bf16 shadow copy, reading the hyper-parameters from device memory so that the launch can be
replayed from a CUDA graph while the learning rate and step count change.

Complex parameters are stored as complex64 and updated through their interleaved real view.
`complex_mode="split"` (default) treats real and imaginary parts as independent reals: that is stock
`torch.optim.AdamW`, which the reference's trainer instantiates (makani/utils/trainer.py:426-433).
`complex_mode="modulus"` shares |g|^2 between the two parts, the convention of the patched optimisers the reference
ships but does not use (makani/third_party/torch/optim/adam.py:391).
"""

from __future__ import annotations

import math
import struct
from typing import Iterable, List, Optional

import torch

from . import _ext

_CHUNK = 1 << 16


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, adamw: bool = True,
                 complex_mode: str = "split", grad_scale: float = 1.0):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adamw = adamw
        self.complex_mode = complex_mode
        self.grad_scale = grad_scale
        self._tables = {}
        self._step_count = 0

    # ---- state helpers -------------------------------------------------------------------------------
    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["step"] = torch.zeros((), dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    @staticmethod
    def _real(t):
        return torch.view_as_real(t) if t.is_complex() else t

    def _build_table(self, gi, group, plist):
        ext = _ext.require()
        dev = plist[0].device
        rows, chunk_tensor, chunk_off = [], [], []
        for ti, p in enumerate(plist):
            st = self._init_state(p)
            pr, gr = self._real(p.data), self._real(p.grad)
            m, v = self._real(st["exp_avg"]), self._real(st["exp_avg_sq"])
            assert pr.is_contiguous() and gr.is_contiguous(), "fused AdamW needs contiguous params and grads"
            n = pr.numel()
            pair = 1 if (p.is_complex() and self.complex_mode == "modulus") else 0
            wd_scale = 0.0 if getattr(p, "_no_weight_decay", False) else 1.0
            packed = struct.unpack("<q", struct.pack("<fi", wd_scale, pair))[0]
            shadow = getattr(p, "_bf16_shadow", None)
            rows.append([pr.data_ptr(), gr.data_ptr(), m.data_ptr(), v.data_ptr(),
                         shadow.data_ptr() if shadow is not None else 0, n, packed])
            for off in range(0, n, _CHUNK):
                chunk_tensor.append(ti)
                chunk_off.append(off)
        assert ext.adam_entry_bytes() == 56
        table = torch.tensor(rows, dtype=torch.int64, device=dev)
        ct = torch.tensor(chunk_tensor, dtype=torch.int32, device=dev)
        co = torch.tensor(chunk_off, dtype=torch.int64, device=dev)
        hyper = torch.zeros(8, dtype=torch.float32, device=dev)
        sig = tuple((p.data_ptr(), p.grad.data_ptr()) for p in plist)
        return dict(table=table, ct=ct, co=co, hyper=hyper, sig=sig)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.prepare_step()
        self.launch_step()
        return loss

    # The update is split in two so that the kernel launches can live inside a CUDA graph: `prepare_step` advances
    # the step counters and uploads the hyper-parameters (host work, outside the graph); `launch_step` only
    # launches kernels that read them from device memory.
    def _groups_with_grads(self):
        for gi, group in enumerate(self.param_groups):
            plist = [p for p in group["params"] if p.grad is not None]
            if plist:
                yield gi, group, plist

    def prepare_step(self):
        from .spectral import note_weights_changed
        note_weights_changed()      # also covers updates replayed from a CUDA graph, which never re-enter `launch_step`
        self._step_count += 1
        self._prepared = True
        for gi, group, plist in self._groups_with_grads():
            if not plist[0].is_cuda:
                continue          # the CPU path keeps its own step counters
            tb = self._table_for(gi, group, plist)
            for p in plist:
                self.state[p]["step"] += 1
            step = float(self.state[plist[0]]["step"])
            b1, b2 = group["betas"]
            host = tb.get("hyper_host")
            if host is None:
                host = tb["hyper_host"] = torch.zeros(8, dtype=torch.float32).pin_memory()
            # the pinned staging vector is reused: wait for the previous upload before overwriting it
            ev = tb.get("hyper_ev")
            if ev is not None:
                ev.synchronize()
            host.copy_(torch.tensor([group["lr"], b1, b2, group["eps"], group["weight_decay"], step, self.grad_scale,
                                     1.0 if self.adamw else 0.0], dtype=torch.float32))
            tb["hyper"].copy_(host, non_blocking=True)
            ev = tb["hyper_ev"] = torch.cuda.Event()
            ev.record()

    def prepare_tables(self):
        """Builds the device-side pointer tables (host-to-device copies) ahead of a stream capture; gradients must
        exist already."""
        for gi, group, plist in self._groups_with_grads():
            if plist[0].is_cuda:
                self._table_for(gi, group, plist)

    def launch_step(self):
        from .spectral import note_weights_changed
        note_weights_changed()      # the kernels write parameters through raw pointers: derived caches are stale now
        for gi, group, plist in self._groups_with_grads():
            if plist[0].is_cuda:
                tb = self._table_for(gi, group, plist)
                _ext.require().adamw_step(tb["table"], tb["ct"], tb["co"], _CHUNK, tb["hyper"])
            else:
                self._step_torch(group, plist)

    def _table_for(self, gi, group, plist):
        sig = tuple((p.data_ptr(), p.grad.data_ptr()) for p in plist)
        tb = self._tables.get(gi)
        if tb is None or tb["sig"] != sig:
            tb = self._build_table(gi, group, plist)
            self._tables[gi] = tb
        return tb

    def _step_torch(self, group, plist):
        b1, b2 = group["betas"]
        lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
        for p in plist:
            st = self._init_state(p)
            st["step"] += 1
            step = float(st["step"])
            g = p.grad * self.grad_scale
            wdp = 0.0 if getattr(p, "_no_weight_decay", False) else wd
            if self.adamw:
                p.mul_(1.0 - lr * wdp)
            else:
                g = g + wdp * p
            m, v = st["exp_avg"], st["exp_avg_sq"]
            m.mul_(b1).add_(g, alpha=1.0 - b1)
            if p.is_complex():
                if self.complex_mode == "modulus":
                    g2 = (g * g.conj()).real
                    vr = torch.view_as_real(v)
                    vr.mul_(b2).add_(torch.stack([g2, g2], dim=-1), alpha=1.0 - b2)
                else:
                    gr = torch.view_as_real(g)
                    torch.view_as_real(v).mul_(b2).add_(gr * gr, alpha=1.0 - b2)
                denom = torch.view_as_real(v).sqrt() / math.sqrt(1.0 - b2 ** step) + eps
                upd = torch.view_as_real(m) / denom
                torch.view_as_real(p).add_(upd, alpha=-lr / (1.0 - b1 ** step))
            else:
                v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
                denom = v.sqrt() / math.sqrt(1.0 - b2 ** step) + eps
                p.addcdiv_(m, denom, value=-lr / (1.0 - b1 ** step))


class LAMB(torch.optim.Optimizer):
    """Layer-wise adaptive moments (You et al., 2020), the update rule of apex `FusedLAMB` that the reference offers
    as `optimizer_type: FusedLAMB` (makani/utils/trainer.py:434-448), written with multi-tensor (`_foreach`) ops so that
    it needs no extra dependency and runs on CPU and GPU alike.

        m = b1 m + (1 - b1) g          v = b2 v + (1 - b2) g^2          (g clipped to a global norm of `max_grad_norm`)
        u = m_hat / (sqrt(v_hat) + eps) + wd * p        p -= lr * (||p|| / ||u||) * u      (trust ratio 1 if a norm is 0)

    Complex parameters are updated through their interleaved real view.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, bias_correction=True,
                 max_grad_norm=1.0, use_nvlamb=False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, bias_correction=bias_correction,
                        max_grad_norm=max_grad_norm)
        super().__init__(params, defaults)
        self.use_nvlamb = use_nvlamb      # apply the trust ratio also to parameters without weight decay

    @staticmethod
    def _real(t):
        return torch.view_as_real(t) if t.is_complex() else t

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # global gradient norm over all groups (fp32)
        grads = [self._real(p.grad) for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not grads:
            return loss
        gnorm = torch.linalg.vector_norm(torch.stack(torch._foreach_norm(grads)))
        for group in self.param_groups:
            plist = [p for p in group["params"] if p.grad is not None]
            if not plist:
                continue
            b1, b2 = group["betas"]
            clip = torch.clamp(gnorm / group["max_grad_norm"], min=1.0) if group["max_grad_norm"] > 0 else torch.ones_like(gnorm)
            ps, gs, ms, vs = [], [], [], []
            for p in plist:
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(self._real(p))
                    st["exp_avg_sq"] = torch.zeros_like(self._real(p))
                st["step"] += 1
                ps.append(self._real(p))
                gs.append(self._real(p.grad))
                ms.append(st["exp_avg"])
                vs.append(st["exp_avg_sq"])
            step = self.state[plist[0]]["step"]
            gs = torch._foreach_div(gs, clip)
            torch._foreach_mul_(ms, b1)
            torch._foreach_add_(ms, gs, alpha=1.0 - b1)
            torch._foreach_mul_(vs, b2)
            torch._foreach_addcmul_(vs, gs, gs, value=1.0 - b2)
            bc1 = 1.0 - b1 ** step if group["bias_correction"] else 1.0
            bc2 = 1.0 - b2 ** step if group["bias_correction"] else 1.0
            denom = torch._foreach_sqrt(torch._foreach_div(vs, bc2))
            torch._foreach_add_(denom, group["eps"])
            upd = torch._foreach_div(torch._foreach_div(ms, bc1), denom)
            wd = group["weight_decay"]
            if wd != 0.0:
                torch._foreach_add_(upd, ps, alpha=wd)
            pn = torch._foreach_norm(ps)
            un = torch._foreach_norm(upd)
            for p_, u_, a, b in zip(ps, upd, pn, un):
                if wd != 0.0 or self.use_nvlamb:
                    ratio = torch.where((a > 0) & (b > 0), a / b, torch.ones_like(a))
                else:
                    ratio = torch.ones_like(a)
                p_.add_(u_ * ratio, alpha=-group["lr"])
        return loss
