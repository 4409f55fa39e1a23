"""A gated delta rule with one decay per key channel, as a mixer with per-sequence state.

    q = Wq x1, k = Wk x1  (kv_heads x dim),   v = Wv x1  (heads x vdim);   head h reads key head h / (heads / kv_heads)
    each passes a short causal convolution over time (per channel, ``taps`` wide, zeros before the start), then silu
    q, k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dim^-1/2
    beta = sigmoid(Wb x1)  per head;    g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 x1) + dt_bias))  per head and key channel
    per head:  S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
    out = Wo (o / rms_head(o) * norm * sigmoid(Wg2 (Wg1 x1)))

S is zero when a sequence starts, float, and carried from step to step together with the last ``taps - 1`` inputs
of the convolutions in the engine's per-sequence state (one row per slot).  Decays, their logarithms and
exponentials, beta, the unit norms, the state and the per-head norm are float on both paths; the bfloat16 path
differs in the type of the projections' results.  The projections of beta and of the decay write float (their
error would add up along the sequence).  Kernels: csrc/channel_delta.cu.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import MIXERS, Mixer, ParamDecl, StateNeed
from .linear import matmul_nt


@MIXERS.register("channel_delta")
class ChannelDelta(Mixer):
    """params: width, heads, kv_heads, dim, vdim, taps, decay_rank, gate_rank, eps."""
    graph_safe = True
    launches_only = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        g = lambda n: int(params[n])
        self.d, self.H, self.G, self.dim, self.vdim = g("width"), g("heads"), g("kv_heads"), g("dim"), g("vdim")
        self.taps, self.ra, self.rg = g("taps"), g("decay_rank"), g("gate_rank")
        self.eps = float(params["eps"])
        if self.H % self.G:
            raise ValueError(f"{self.H} heads cannot share {self.G} key heads")
        if self.dim > 256:
            raise ValueError(f"the delta-rule kernel takes heads of up to 256 query/key entries, got {self.dim}")
        if not (1 <= self.taps <= 16):
            raise ValueError(f"the convolution takes 1 to 16 taps, got {self.taps}")
        self.hk, self.hv = self.G * self.dim, self.H * self.vdim
        self.C = 2 * self.hk + self.hv                       # channels that pass the convolution: q, k, v
        self.z_width = self.C + self.ra + self.rg

    def parameters(self):
        return {
            "win": ParamDecl((self.z_width, self.d)),              # rows: q, k, v, the decay's and the gate's first
            "conv": ParamDecl((self.C, self.taps), "norm", "normal"),
            "wb": ParamDecl((self.H, self.d)),
            "a2": ParamDecl((self.H * self.dim, self.ra)),
            "g2": ParamDecl((self.hv, self.rg)),
            "dt_bias": ParamDecl((self.H * self.dim,), "norm", "normal"),
            "A_log": ParamDecl((self.H,), "norm", "normal"),
            "norm": ParamDecl((self.vdim,), "norm", "ones"),
            "wo": ParamDecl((self.d, self.hv)),
        }

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # the kernel that norms the heads' outputs takes one weight per (head, entry): the shared one, repeated
        self.weights["norm"] = self.weights["norm"].float().repeat(self.H).contiguous()

    def state_need(self):
        return StateNeed((lib.delta_state_size(self.G, self.H, self.dim, self.vdim, self.taps),), torch.float32)

    def forward(self, ctx, x1, out, cache, state) -> None:
        nt, H = x1.shape[0], self.H
        sfx = lib.suffix(self.dtype)
        w = self.weights
        z = ctx.scratch("delta.z", (nt, self.z_width), self.dtype)
        matmul_nt(x1, w["win"], z)
        bz = ctx.scratch("delta.bz", (nt, H), torch.float32)
        matmul_nt(x1, w["wb"], bz)                                          # float out on both paths
        a = ctx.scratch("delta.a", (nt, H * self.dim), torch.float32)
        matmul_nt(z[:, self.C:self.C + self.ra], w["a2"], a)               # float out
        gz = ctx.scratch("delta.gz", (nt, self.hv), self.dtype)
        matmul_nt(z[:, self.C + self.ra:], w["g2"], gz)
        # what enters the recurrence, float: one record per (token, head) [q | k | decay | beta, k.q], and the values
        rec = ctx.scratch("delta.rec", (nt, H, lib.delta_record_size(self.dim)), torch.float32)
        vals = ctx.scratch("delta.v", (nt, H, lib.delta_value_pitch(self.vdim)), torch.float32)
        lib.call("tb_delta_prep_" + sfx, lib.ptr(z), self.z_width, lib.ptr(w["conv"]), lib.ptr(state), lib.ptr(a),
                 lib.ptr(w["dt_bias"]), lib.ptr(w["A_log"]), lib.ptr(bz), lib.ptr(rec), lib.ptr(vals),
                 lib.ptr(ctx.tok_seq), lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), nt, ctx.B, self.G, H,
                 self.dim, self.vdim, self.taps, 1 if ctx.decode else 0)
        o = ctx.scratch("delta.o", (nt, self.hv), torch.float32)
        lib.call("tb_delta_scan", lib.ptr(rec), lib.ptr(vals), lib.ptr(state), lib.ptr(o),
                 lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), nt, ctx.B, self.G, H, self.dim, self.vdim, self.taps)
        y = ctx.scratch("delta.y", (nt, self.hv), self.dtype)
        lib.call("tb_mlstm_out_" + sfx, lib.ptr(o), lib.ptr(gz), self.hv, lib.ptr(w["norm"]), lib.ptr(y), nt, H,
                 self.vdim, self.eps)
        matmul_nt(y, w["wo"], out)
