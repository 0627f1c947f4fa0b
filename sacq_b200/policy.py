"""Synthetic GR00T-N1.5-shaped policy forward with every linear at W1.5A8.

A shape-equivalent stand-in, not the GR00T model: the reference's model sources
(``gr00t.model.modules.dit``, the Qwen3 backbone) are not part of its tree and no
checkpoint is available, so weights are random and no action parity is claimed.  What it
reproduces is the *workload* a policy query puts on the quantized-linear path:

  * vision tower: 24 pre-norm transformer blocks, hidden 1024, MLP 4096, 256 patch tokens;
  * language model: 12 blocks, hidden 2048, 16 query / 8 key-value heads of 128, gated MLP
    6144, 300 prefill tokens (the first 256 are the projected patch tokens);
  * action head: 16 DiT blocks, hidden 1536, self-attention over the 16-step action
    horizon, cross-attention to the language tokens, MLP 6144, AdaLN timestep modulation,
    4 Euler flow-matching steps (the loop structure of gr00t_n1d7.py:396-434).

Attention uses stock PyTorch; norms, AdaLN modulation, activation functions and residual
adds run inside this library's quantizer and GEMM kernels; every projection is a
``PrecomputedPackedVectorCodebookLinear`` (dim-8 vectors, 4096-entry codebook,
per-output-channel scales).  The cross-attention keys/values depend only on the language
tokens and are computed once per query, not once per denoising step.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .activation import act_quantize_rows, layernorm_quantize_rows, quantize_rows
from .linear import PrecomputedPackedVectorCodebookLinear, forward_shared, linear_a8_multi
from .synthetic import make_payload


class _Factory:
    """Creates quantized linears with seeded random payloads (one fitted payload per shape;
    layers of the same shape get their own device buffers)."""

    def __init__(self, device: torch.device, seed: int):
        self.device = device
        self.seed = seed
        self._payloads = {}
        self.count = 0

    def linear(self, k: int, n: int) -> PrecomputedPackedVectorCodebookLinear:
        key = (k, n)
        if key not in self._payloads:
            self._payloads[key] = make_payload(n, k, seed=self.seed + len(self._payloads), device=self.device,
                                               fit=False)
        self.count += 1
        return PrecomputedPackedVectorCodebookLinear(self._payloads[key], None, str(self.device))


class _Block(torch.nn.Module):
    """Pre-norm transformer block: self-attention (+ optional cross-attention) + MLP."""

    def __init__(self, f: _Factory, hidden: int, heads: int, kv_heads: int, mlp: int, gated: bool,
                 cross_dim: int | None = None, adaln: bool = False):
        super().__init__()
        self.hidden, self.heads, self.kv_heads = hidden, heads, kv_heads
        self.head_dim = hidden // heads
        kv = kv_heads * self.head_dim
        self.q, self.k, self.v, self.o = f.linear(hidden, hidden), f.linear(hidden, kv), f.linear(hidden, kv), \
            f.linear(hidden, hidden)
        self.gated = gated
        if gated:
            self.gate, self.up = f.linear(hidden, mlp), f.linear(hidden, mlp)
        else:
            self.up = f.linear(hidden, mlp)
        self.down = f.linear(mlp, hidden)
        self.cross = cross_dim is not None
        if self.cross:
            self.cq, self.ck, self.cv, self.co = f.linear(hidden, hidden), f.linear(cross_dim, hidden), \
                f.linear(cross_dim, hidden), f.linear(hidden, hidden)
        self.adaln = adaln
        if adaln:
            self.mod = f.linear(hidden, 4 * hidden)          # shift and scale for the two modulated norms
        self.n1 = torch.nn.LayerNorm(hidden, elementwise_affine=not adaln, device=f.device, dtype=torch.bfloat16)
        self.n2 = torch.nn.LayerNorm(hidden, elementwise_affine=not adaln, device=f.device, dtype=torch.bfloat16)
        if self.cross:
            self.n3 = torch.nn.LayerNorm(hidden, device=f.device, dtype=torch.bfloat16)

    def _attend(self, q, k, v, batch=1):
        # [batch, heads, tokens, head_dim] views: the 4-D form lets PyTorch pick a fused attention
        # kernel, and grouped-query attention needs no materialised key/value repeats; the rows
        # of q, k, v are request-major, so every request attends to its own tokens only
        t, s = q.shape[0] // batch, k.shape[0] // batch
        q = q.view(batch, t, self.heads, self.head_dim).transpose(1, 2)
        k = k.view(batch, s, -1, self.head_dim).transpose(1, 2)
        v = v.view(batch, s, -1, self.head_dim).transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v, enable_gqa=k.shape[1] != self.heads)
        return out.transpose(1, 2).reshape(batch * t, self.hidden)

    def cross_kv(self, ctx):
        return tuple(forward_shared((self.ck, self.cv), ctx))

    def _norm_quant(self, norm, x, scale=None, shift=None):
        """LayerNorm (+ AdaLN modulation) inside the quantizer of the projections it feeds."""
        return layernorm_quantize_rows(x, norm.weight, norm.bias, norm.eps, mod_scale=scale, mod_shift=shift)

    def forward(self, x, cond=None, cross_kv=None, modulation=None, batch=1):
        if self.adaln:
            m = (self.mod(cond) if modulation is None else modulation).view(4, self.hidden)
        else:
            m = (None,) * 4
        qa, sa = self._norm_quant(self.n1, x, m[1], m[0])
        q, k, v = linear_a8_multi((self.q, self.k, self.v), qa, sa)        # one launch for q/k/v at small M
        x = self.o.forward_residual(self._attend(q, k, v, batch), x)     # residual added in the GEMM epilogue
        if self.cross:
            qc, sc = self._norm_quant(self.n3, x)
            x = self.co.forward_residual(self._attend(self.cq.linear_a8(qc, sc), cross_kv[0], cross_kv[1], batch), x)
        qu, su = self._norm_quant(self.n2, x, m[3], m[2])
        # the activation function runs inside the quantizer of the down projection
        if self.gated:
            gate, up = linear_a8_multi((self.gate, self.up), qu, su)
            qd, sd = act_quantize_rows("silu_mul", gate, up)
        else:
            qd, sd = act_quantize_rows("gelu", self.up.linear_a8(qu, su))
        return self.down.linear_a8(qd, sd, residual=x)


class SyntheticGr00tPolicy(torch.nn.Module):
    VIT_LAYERS, VIT_HIDDEN, VIT_MLP, PATCHES = 24, 1024, 4096, 256
    LLM_LAYERS, LLM_HIDDEN, LLM_MLP, LLM_TOKENS = 12, 2048, 6144, 300
    DIT_LAYERS, DIT_HIDDEN, DIT_MLP, HORIZON, STEPS = 16, 1536, 6144, 16, 4
    ACTION_DIM = 32
    BENCH_BATCH = 64          # independent requests per forward in the batched-throughput measurement

    def __init__(self, device: str = "cuda", seed: int = 0):
        super().__init__()
        dev = torch.device(device)
        f = _Factory(dev, seed)
        g = torch.Generator().manual_seed(seed)
        bf = dict(device=dev, dtype=torch.bfloat16)
        self.patch_embed = (torch.randn(3 * 14 * 14, self.VIT_HIDDEN, generator=g) * 0.02).to(**bf)
        self.vit = torch.nn.ModuleList(_Block(f, self.VIT_HIDDEN, 16, 16, self.VIT_MLP, gated=False)
                                       for _ in range(self.VIT_LAYERS))
        self.vis_proj = f.linear(self.VIT_HIDDEN, self.LLM_HIDDEN)
        self.text_embed = (torch.randn(self.LLM_TOKENS - self.PATCHES, self.LLM_HIDDEN, generator=g) * 0.02).to(**bf)
        self.llm = torch.nn.ModuleList(_Block(f, self.LLM_HIDDEN, 16, 8, self.LLM_MLP, gated=True)
                                       for _ in range(self.LLM_LAYERS))
        self.dit = torch.nn.ModuleList(_Block(f, self.DIT_HIDDEN, 12, 12, self.DIT_MLP, gated=False,
                                              cross_dim=self.LLM_HIDDEN, adaln=True) for _ in range(self.DIT_LAYERS))
        self.time_embed = (torch.randn(self.STEPS, self.DIT_HIDDEN, generator=g) * 0.02).to(**bf)
        self.action_in = (torch.randn(self.ACTION_DIM, self.DIT_HIDDEN, generator=g) * 0.02).to(**bf)
        self.action_out = (torch.randn(self.DIT_HIDDEN, self.ACTION_DIM, generator=g) * 0.02).to(**bf)
        self.num_quantized_linears = f.count
        self.device = dev

    def quantized_linear_calls_per_query(self) -> int:
        vit = self.VIT_LAYERS * 6
        llm = self.LLM_LAYERS * 7
        dit = self.DIT_LAYERS * (2 + self.STEPS * 9)       # cross K/V once, 9 projections per step
        return vit + 1 + llm + dit

    @torch.no_grad()
    def forward(self, image: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
        """image: [3, 224, 224] bf16 and noise: [HORIZON, ACTION_DIM] bf16 -> actions [HORIZON, ACTION_DIM];
        or a batch of B independent requests, image [B, 3, 224, 224] and noise [B, HORIZON, ACTION_DIM]
        -> [B, HORIZON, ACTION_DIM].  The requests of a batch share nothing but the weights: their
        tokens are stacked along the row dimension of every linear (M = B x tokens) and attention
        runs per request."""
        single = image.dim() == 3
        if single:
            image, noise = image.unsqueeze(0), noise.unsqueeze(0)
        b = image.shape[0]
        patches = image.unfold(2, 14, 14).unfold(3, 14, 14).permute(0, 2, 3, 1, 4, 5).reshape(b * self.PATCHES, -1)
        x = patches @ self.patch_embed
        for blk in self.vit:
            x = blk(x, batch=b)
        vis = self.vis_proj(x).view(b, self.PATCHES, self.LLM_HIDDEN)
        tokens = torch.cat([vis, self.text_embed.unsqueeze(0).expand(b, -1, -1)], dim=1).reshape(-1, self.LLM_HIDDEN)
        for blk in self.llm:
            tokens = blk(tokens, batch=b)
        kv = [blk.cross_kv(tokens) for blk in self.dit]
        # the AdaLN modulation vectors depend on the denoising step only: all blocks' modulation
        # layers read the same one-row input, so they run four to a launch, ahead of the loop
        mods = []
        for step in range(self.STEPS):
            qc, sc = quantize_rows(self.time_embed[step: step + 1])
            per_block = []
            for i in range(0, len(self.dit), 4):
                per_block += linear_a8_multi([blk.mod for blk in self.dit[i: i + 4]], qc, sc)
            mods.append(per_block)
        actions = noise.reshape(b * self.HORIZON, self.ACTION_DIM)
        dt = 1.0 / self.STEPS
        for step in range(self.STEPS):
            h = actions @ self.action_in
            for blk, ckv, mod in zip(self.dit, kv, mods[step]):
                h = blk(h, cross_kv=ckv, modulation=mod, batch=b)
            actions = actions + dt * (h @ self.action_out)
        actions = actions.view(b, self.HORIZON, self.ACTION_DIM)
        return actions[0] if single else actions

    def example_inputs(self, seed: int = 42, batch: int = 1):
        """Seeded inputs: one request ([3, 224, 224], [HORIZON, ACTION_DIM]) for batch = 1, else
        a batch of distinct requests with a leading batch dimension."""
        g = torch.Generator().manual_seed(seed)
        image = torch.rand(batch, 3, 224, 224, generator=g).to(device=self.device, dtype=torch.bfloat16)
        noise = torch.randn(batch, self.HORIZON, self.ACTION_DIM, generator=g).to(device=self.device,
                                                                                  dtype=torch.bfloat16)
        return (image[0], noise[0]) if batch == 1 else (image, noise)
