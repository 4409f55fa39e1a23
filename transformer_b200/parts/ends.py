"""The two ends of the model: token ids into the residual stream, normed rows into logits.

The reference's caller gathers embedding rows (models/llama/cuda/src/infer.rs:98-104,
test-utils/src/llama.rs:18-23) and its step ends with ``logits = x . output`` on the wanted rows
(models/llama/common/src/compute.rs:364-365; ``output`` is ``token_embd`` when the file has no
``output.weight``, storage.rs:84).  Here both are parts like any other: a model with a scaled
embedding, learned positions or capped logits registers another kind and the engine stays as it is.
"""
from __future__ import annotations

import torch

from ..csrc import lib
from .base import EMBEDDINGS, HEADS, Embedding, Head, ParamDecl, StateNeed
from .linear import matmul_nt


@EMBEDDINGS.register("lookup")
class Lookup(Embedding):
    """params: vocab, width, scale (default 1).  x[i] = table[tok_i] * scale, in float."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.scale = float(params.get("scale", 1.0))

    def parameters(self):
        return {"table": ParamDecl((self.vocab, self.width))}

    def forward(self, ctx, x) -> None:
        if self.scale != 1.0:
            lib.call("tb_embed_scaled_" + lib.suffix(self.dtype), lib.ptr(ctx.tok_ids), lib.ptr(self.weights["table"]),
                     lib.ptr(x), x.shape[0], self.width, self.scale)
            return
        lib.call("tb_embed_" + lib.suffix(self.dtype), lib.ptr(ctx.tok_ids), lib.ptr(self.weights["table"]),
                 lib.ptr(x), x.shape[0], self.width)


@EMBEDDINGS.register("bigram_lookup")
class BigramLookup(Embedding):
    """params: vocab, width, scale, buckets, mul_prev, mul_cur.

        x[i] = table[tok_i] * scale + pairs[(tok_{i-1} * mul_prev + tok_i * mul_cur) mod buckets]

    in float; a sequence's first token takes the last row of ``pairs`` (row ``buckets``).  The token before a step's
    first one is state of the sequence (one int32 per slot), kept on the device, so that steps whose tokens never
    reach the host (a sampler's output fed straight back) and captured graphs see it too."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        g = lambda n: int(params[n])
        self.vocab, self.width, self.buckets = g("vocab"), g("width"), g("buckets")
        self.mul_prev, self.mul_cur = g("mul_prev"), g("mul_cur")
        self.scale = float(params.get("scale", 1.0))
        if self.buckets <= 0:
            raise ValueError(f"the pair table needs at least one bucket, got {self.buckets}")

    def parameters(self):
        return {"table": ParamDecl((self.vocab, self.width)), "pairs": ParamDecl((self.buckets + 1, self.width))}

    def state_need(self):
        return StateNeed((1,), torch.int32)

    def forward(self, ctx, x, state=None) -> None:
        lib.call("tb_embed_bigram_" + lib.suffix(self.dtype), lib.ptr(ctx.tok_ids), lib.ptr(ctx.tok_seq),
                 lib.ptr(ctx.tok_pos), lib.ptr(ctx.seq_start), lib.ptr(ctx.slots), lib.ptr(state),
                 lib.ptr(self.weights["table"]), lib.ptr(self.weights["pairs"]), lib.ptr(x), x.shape[0], self.width,
                 self.scale, self.buckets, self.mul_prev, self.mul_cur)


@HEADS.register("linear")
class LinearHead(Head):
    """params: vocab, width, tied, scale (default 1).  logits = xn weight^T * scale in float, no bias, no cap.
    ``tied``: the weight is the embedding's table unless the file holds one of its own (the weight plan's business,
    not this part's)."""
    graph_safe = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.vocab, self.width = int(params["vocab"]), int(params["width"])
        self.scale = float(params.get("scale", 1.0))

    def parameters(self):
        return {"weight": ParamDecl((self.vocab, self.width))}

    def forward(self, ctx, xn, logits) -> None:
        matmul_nt(xn, self.weights["weight"], logits)
        if self.scale != 1.0:
            lib.call("tb_scale_f32", lib.ptr(logits), logits.numel(), self.scale)
