"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

All tensors are generated on the CPU with an explicit generator in fp32 and cast last, so that the GPU path and
the CPU oracle see identical bits.
"""

from __future__ import annotations

import torch


def normal_with_outliers(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    """N(0,1) with 0.1 % of the entries replaced by N(0,1)*100 (fp32)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    m = torch.rand(rows, cols, generator=g) < 1e-3
    return torch.where(m, torch.randn(rows, cols, generator=g) * 100, x)


def student_t3(rows: int, cols: int, seed: int = 1, scale: float = 0.02, dtype=torch.bfloat16) -> torch.Tensor:
    """Student-t with 3 degrees of freedom times `scale`: z / sqrt(chi2_3 / 3) from seeded normals."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(rows, cols, generator=g)
    chi = torch.zeros(rows, cols)
    for _ in range(3):
        chi += torch.randn(rows, cols, generator=g) ** 2
    return (z / (chi / 3).sqrt() * scale).to(dtype)


def linear_operands(m: int, k: int = 4096, n: int = 4096, seed: int = 2, dtype=torch.bfloat16):
    """W[n,k] ~ N(0, 0.02); x[m,k] ~ N(0,1) with 1 % of the k channels scaled by 50."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    ch = torch.rand(k, generator=g) < 0.01
    x = torch.randn(m, k, generator=g)
    x = torch.where(ch.view(1, -1), x * 50, x)
    return x.to(dtype), w.to(dtype)


def device_student_t3(rows: int, cols: int, seed: int, device, dtype=torch.bfloat16, scale: float = 0.02):
    """The same distribution generated directly on a CUDA device (for tensors too large to stage on the host)."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = torch.empty(rows, cols, dtype=dtype, device=device)
    step = max(1, (1 << 26) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        z = torch.randn(r1 - r0, cols, generator=g, device=device)
        chi = torch.zeros_like(z)
        for _ in range(3):
            chi += torch.randn(r1 - r0, cols, generator=g, device=device) ** 2
        out[r0:r1] = (z / (chi / 3).sqrt() * scale).to(dtype)
    return out


# ---- mixed-precision decoder layer (Llama-style, random weights) ---------------------------------------------------
MXINT8_LINEAR = {"weight_block_size": 32, "weight_width": 8, "data_in_block_size": 32, "data_in_width": 8}
MXFP4W_MXFP8A_LINEAR = {"weight_block_size": 32, "weight_exponent_width": 2, "weight_frac_width": 1,
                        "data_in_block_size": 32, "data_in_exponent_width": 4, "data_in_frac_width": 3}


class DecoderLayer(torch.nn.Module):
    """Pre-norm decoder layer: RMSNorm -> q/k/v -> RoPE -> causal attention -> o -> residual -> RMSNorm -> SwiGLU
    (gate, up, down) -> residual.  The seven projections are `torch.nn.Linear` children without bias, which a
    quantize pass (or `quantize_decoder_layer`) swaps for quantized classes; norms (computed in fp32, weights 1),
    RoPE, softmax and SiLU stay unquantized."""

    ATTENTION = ("q_proj", "k_proj", "v_proj", "o_proj")
    FFN = ("gate_proj", "up_proj", "down_proj")

    def __init__(self, hidden: int = 4096, heads: int = 32, ffn: int = 11008, eps: float = 1e-6, theta: float = 10000.0,
                 seed: int = 3, dtype=torch.bfloat16):
        super().__init__()
        assert hidden % heads == 0
        self.hidden, self.heads, self.ffn, self.eps, self.theta = hidden, heads, ffn, eps, theta
        self._rope_cache = {}
        g = torch.Generator().manual_seed(seed)
        for name, (k, n) in {"q_proj": (hidden, hidden), "k_proj": (hidden, hidden), "v_proj": (hidden, hidden),
                             "o_proj": (hidden, hidden), "gate_proj": (hidden, ffn), "up_proj": (hidden, ffn),
                             "down_proj": (ffn, hidden)}.items():
            lin = torch.nn.Linear(k, n, bias=False, dtype=dtype)
            lin.weight.data.copy_((torch.randn(n, k, generator=g) * 0.02).to(dtype))
            setattr(self, name, lin)

    def _norm(self, x):
        return torch.nn.functional.rms_norm(x, (self.hidden,), None, self.eps)  # fp32 inside, weights 1

    def _rope_tables(self, s, d, device):
        key = (s, d, str(device))
        if self._rope_cache.get("key") != key:
            inv = 1.0 / (self.theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
            ang = torch.arange(s, device=device, dtype=torch.float32)[:, None] * inv[None, :]
            ang = torch.cat([ang, ang], -1)
            self._rope_cache = {"key": key, "cos": ang.cos(), "sin": ang.sin()}
        return self._rope_cache["cos"], self._rope_cache["sin"]

    def _rope(self, t):  # t: [B, heads, S, head_dim]
        s, d = t.shape[-2], t.shape[-1]
        cos, sin = self._rope_tables(s, d, t.device)
        if t.is_cuda:  # one pass over t (the tables are fp32: products and sum in fp32, one rounding)
            from .functional import rope_apply

            out = rope_apply(t, cos, sin)
            if out is not None:
                return out
        rot = torch.cat([-t[..., d // 2:], t[..., : d // 2]], -1)
        return torch.addcmul(t * cos, rot, sin).to(t.dtype)

    def forward(self, x):  # [B, S, hidden]
        b, s, h = x.shape
        hd = h // self.heads
        from .modules import forward_siblings  # plain nn.Linear children simply get called one by one

        y = self._norm(x)
        q, k, v = (t.view(b, s, self.heads, hd).transpose(1, 2)
                   for t in forward_siblings([self.q_proj, self.k_proj, self.v_proj], y))
        q, k = self._rope(q), self._rope(k)
        att = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o_proj(att.transpose(1, 2).reshape(b, s, h))
        y = self._norm(x)
        gate, up = forward_siblings([self.gate_proj, self.up_proj], y)
        if hasattr(self.down_proj, "forward_gated"):
            return x + self.down_proj.forward_gated(gate, up)
        return x + self.down_proj(torch.nn.functional.silu(gate) * up)

    def linear_flops(self, tokens: int) -> int:
        return 2 * tokens * (4 * self.hidden * self.hidden + 3 * self.hidden * self.ffn)


def quantize_decoder_layer(layer: DecoderLayer, make_attention, make_ffn) -> DecoderLayer:
    """Swap the projections the way MASE's module pass does (construct with `config`, then `load_state_dict` of the
    original weights): `make_attention(in, out)` / `make_ffn(in, out)` return the replacement modules."""
    for names, make in ((DecoderLayer.ATTENTION, make_attention), (DecoderLayer.FFN, make_ffn)):
        for name in names:
            old = getattr(layer, name)
            new = make(old.in_features, old.out_features)
            new.load_state_dict(old.state_dict(), strict=False)
            setattr(layer, name, new)
    return layer
