"""CPU oracle for the Qwen3 decode path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this file; it is the checker used by
the tests, by the smoke entry and by the CPU-baseline leg of the benchmark.

Two restatements live here, both on CPU with plain torch ops:

* ``TorchRefModel`` follows the reference's own PyTorch model,
  demo/qwen3/models/modeling_qwen3.py, function by function (citations on
  each method).  It is pinned against the unmodified reference file by
  tests/golden/make_golden.py, which imports the reference model, runs both on
  the same seeded weights and commits the reference's outputs as fixtures.
* the ``mpk_*`` functions restate the arithmetic of the reference's megakernel
  tasks (fp32 maths, one bf16 rounding per task output), which is what the
  CUDA kernels implement.  The two differ only in rounding (the PyTorch model
  normalises in bf16 without eps), far inside the 2e-2 logit tolerance.

Seeded synthetic inputs (weights, prompts, KV cache) are generated here so that
the oracle and the CUDA path always see the same bytes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict

import torch
import torch.nn.functional as F

BF16 = torch.bfloat16


@dataclass(frozen=True)
class Geometry:
    hidden: int = 4096
    n_q: int = 32
    n_kv: int = 8
    head_dim: int = 128
    mlp: int = 12288
    layers: int = 36
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    init_std: float = 0.02

    def asdict(self):
        return asdict(self)

    @property
    def q_per_kv(self):
        return self.n_q // self.n_kv

    @property
    def qkv_out(self):
        return (self.n_q + 2 * self.n_kv) * self.head_dim


QWEN3_8B = Geometry()
# Small geometries for fast parity cases (head_dim stays 128, as in every Qwen3).
TINY = Geometry(hidden=512, n_q=4, n_kv=2, mlp=1024, layers=3, vocab=2048)
SMALL = Geometry(hidden=1024, n_q=8, n_kv=2, mlp=3072, layers=4, vocab=8192)
# Eight kv heads, so that the model still splits over 2, 4 and 8 tensor-parallel ranks.
KV8 = Geometry(hidden=1024, n_q=16, n_kv=8, mlp=3072, layers=3, vocab=8192)


# ---------------------------------------------------------------------------
# seeded synthetic inputs
# ---------------------------------------------------------------------------
def weight_names(geom: Geometry):
    """Fixed generation order: embedding, per layer q,k,v,o,gate,up,down, LM head."""
    names = [("embed", (geom.vocab, geom.hidden))]
    for i in range(geom.layers):
        names += [
            (f"l{i}.q", (geom.n_q * geom.head_dim, geom.hidden)),
            (f"l{i}.k", (geom.n_kv * geom.head_dim, geom.hidden)),
            (f"l{i}.v", (geom.n_kv * geom.head_dim, geom.hidden)),
            (f"l{i}.o", (geom.hidden, geom.n_q * geom.head_dim)),
            (f"l{i}.gate", (geom.mlp, geom.hidden)),
            (f"l{i}.up", (geom.mlp, geom.hidden)),
            (f"l{i}.down", (geom.hidden, geom.mlp)),
        ]
    names.append(("lm_head", (geom.vocab, geom.hidden)))
    return names


def make_weights(geom: Geometry, seed: int = 0, device: str = "cpu", norm_jitter: float = 0.0):
    """bf16 weights ~ N(0, init_std) drawn in fp32 then rounded, in the order of
    ``weight_names``; every RMSNorm weight is 1.0 (as the reference's
    ``_init_weights`` leaves it, modeling_qwen3.py:47,404-413) unless
    ``norm_jitter`` asks for 1 + U(-j, j) to exercise the norm weights."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in weight_names(geom):
        t = torch.randn(shape, generator=g, dtype=torch.float32, device=device)
        w[name] = (t * geom.init_std).to(BF16)
        del t

    def norm(n):
        if norm_jitter == 0.0:
            return torch.ones(n, dtype=BF16, device=device)
        u = torch.rand(n, generator=g, dtype=torch.float32, device=device)
        return (1.0 + norm_jitter * (2 * u - 1)).to(BF16)

    for i in range(geom.layers):
        w[f"l{i}.ln1"] = norm(geom.hidden)
        w[f"l{i}.ln2"] = norm(geom.hidden)
        w[f"l{i}.qn"] = norm(geom.head_dim)
        w[f"l{i}.kn"] = norm(geom.head_dim)
    w["norm"] = norm(geom.hidden)
    return w


def rope_tables(geom: Geometry, max_pos: int, device: str = "cpu"):
    """cos/sin tables as the reference builds them (modeling_qwen3.py:95-117):
    inv_freq = theta^(-2i/d), emb = cat(freqs, freqs), fp32 cos/sin -> bf16."""
    d = geom.head_dim
    inv_freq = 1.0 / (geom.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    pos = torch.arange(max_pos, dtype=torch.float32)
    freqs = pos[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(BF16).to(device), emb.sin().to(BF16).to(device)


def make_prompt(geom: Geometry, length: int, request: int = 0):
    """Uniform-random token ids, per-request seed 1000 + r."""
    g = torch.Generator().manual_seed(1000 + request)
    return torch.randint(0, geom.vocab, (length,), generator=g, dtype=torch.int64)


# ---------------------------------------------------------------------------
# restatement of the reference PyTorch model
# ---------------------------------------------------------------------------
def ref_rmsnorm(x, w):
    """Qwen3RMSNorm.forward, modeling_qwen3.py:49-54: no eps, no upcast."""
    variance = x.pow(2).mean(-1, keepdim=True)
    x = x * torch.rsqrt(variance)
    return w * x


def ref_rotate_half(x):
    """modeling_qwen3.py:121-125"""
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def ref_rope(q, k, cos, sin, unsqueeze_dim):
    """apply_rotary_pos_emb, modeling_qwen3.py:129-134 (same maths as the Triton
    kernel the GPU path of the reference uses, rope.py:79-80)."""
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (ref_rotate_half(q) * sin), (k * cos) + (ref_rotate_half(k) * sin)


class TorchRefModel:
    """Batch-1 restatement of Qwen3ForCausalLM (modeling_qwen3.py:416-567) with
    its contiguous one-page KV cache (:425-446)."""

    def __init__(self, geom: Geometry, weights: dict, max_seq: int, layers: int | None = None, device: str = "cpu"):
        """``device``: where the torch ops run.  "cpu" is the oracle; "cuda" runs the very same ops
        through torch's GPU libraries (the reference's own GPU PyTorch path), which the tests use as a
        second opinion on how far two executions of the reference model drift apart."""
        self.g = geom
        self.w = weights
        self.device = device
        self.n_layers = geom.layers if layers is None else layers
        self.max_seq = max_seq
        self.k_cache = torch.zeros(self.n_layers, max_seq, geom.n_kv, geom.head_dim, dtype=BF16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(geom, max_seq, device)

    # Qwen3Attention.forward, modeling_qwen3.py:263-337
    def _attention(self, i, h, pos0):
        g, w = self.g, self.w
        q_len = h.shape[0]
        hn = ref_rmsnorm(h, w[f"l{i}.ln1"])
        q = F.linear(hn, w[f"l{i}.q"]).view(1, q_len, g.n_q, g.head_dim)
        k = F.linear(hn, w[f"l{i}.k"]).view(1, q_len, g.n_kv, g.head_dim)
        v = F.linear(hn, w[f"l{i}.v"]).view(1, q_len, g.n_kv, g.head_dim)
        q = ref_rmsnorm(q, w[f"l{i}.qn"])
        k = ref_rmsnorm(k, w[f"l{i}.kn"])
        cos = self.cos[None, pos0:pos0 + q_len]
        sin = self.sin[None, pos0:pos0 + q_len]
        q, k = ref_rope(q, k, cos, sin, unsqueeze_dim=2)
        self.k_cache[i, pos0:pos0 + q_len] = k[0]
        self.v_cache[i, pos0:pos0 + q_len] = v[0]
        kv_len = pos0 + q_len
        # naive_attention, modeling_qwen3.py:168-189
        kk = self.k_cache[i, :kv_len].permute(1, 0, 2)
        vv = self.v_cache[i, :kv_len].permute(1, 0, 2)
        qq = q[0].permute(1, 0, 2)
        o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=(q_len > 1), enable_gqa=True)
        o = o.permute(1, 0, 2).reshape(q_len, g.n_q * g.head_dim)
        return F.linear(o, w[f"l{i}.o"])

    # Qwen3MLP.forward, modeling_qwen3.py:155-166
    def _mlp(self, i, h):
        w = self.w
        hn = ref_rmsnorm(h, w[f"l{i}.ln2"])
        return F.linear(F.silu(F.linear(hn, w[f"l{i}.gate"])) * F.linear(hn, w[f"l{i}.up"]), w[f"l{i}.down"])

    # Qwen3DecoderLayer.forward, modeling_qwen3.py:359-398
    def layer(self, i, h, pos0):
        h = h + self._attention(i, h, pos0)
        h = h + self._mlp(i, h)
        return h

    @torch.inference_mode()
    def forward_hidden(self, h, pos0):
        for i in range(self.n_layers):
            h = self.layer(i, h, pos0)
        return h

    # Qwen3Model.forward + Qwen3ForCausalLM.forward, modeling_qwen3.py:473-505, 543-567
    @torch.inference_mode()
    def forward(self, token_ids, pos0):
        h = F.embedding(token_ids.to(self.device), self.w["embed"])
        h = self.forward_hidden(h, pos0)
        h = ref_rmsnorm(h, self.w["norm"])
        return F.linear(h, self.w["lm_head"])

    @torch.inference_mode()
    def generate(self, prompt, n_new, forced=None, one_token_prefill=False):
        """Greedy decode as demo/qwen3/demo.py:1196-1212 drives the model: one
        multi-token prefill call, then one token per call.  Returns (tokens,
        logits[n_new, vocab]) where logits[j] produced generated token j.
        ``forced`` (teacher forcing): token ids fed instead of the argmax."""
        toks = prompt.clone().tolist()
        P = len(toks)
        logits_out = []
        if one_token_prefill:
            for p in range(P):
                lg = self.forward(torch.tensor([toks[p]]), p)
        else:
            lg = self.forward(torch.tensor(toks), 0)
        for j in range(n_new):
            last = lg[-1]
            logits_out.append(last.clone().cpu())
            nxt = int(last.argmax(-1))
            toks.append(nxt if forced is None else int(forced[j]))
            if j + 1 < n_new:
                lg = self.forward(torch.tensor([toks[-1]]), P + j)
        return toks, torch.stack(logits_out)


# ---------------------------------------------------------------------------
# restatement of the megakernel tasks' arithmetic (what the CUDA kernels do)
# ---------------------------------------------------------------------------
def mpk_rmsnorm(x, w, eps=1e-6):
    """tasks/hopper/rmsnorm_hopper.cuh:106-137: fp32 sum of squares,
    rsqrt(mean + eps), val * (rms_rcp * w), one rounding to bf16."""
    xf = x.float()
    r = torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * (r * w.float())).to(BF16)


def mpk_linear(x, w, residual=None):
    """tasks/blackwell/linear_sm100_mpk.cuh:623-661: fp32 accumulate, residual
    added in fp32, one rounding to bf16."""
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return y.to(BF16)


def mpk_silu_mul(gate, up):
    """tasks/ampere/silu_mul.cuh:37-40: bf16(x / (1 + exp(-x))) * up in bf16."""
    gf = gate.float()
    s = (gf / (1.0 + torch.exp(-gf))).to(BF16)
    return s * up


def mpk_qk_norm_rope(x, w, cos, sin, eps=1e-6):
    """tasks/blackwell/norm_sm100.cuh:66-126 for one head vector x[..., d]:
    fp32 RMSNorm -> bf16, then rotate-half RoPE in fp32 from bf16 cos/sin -> bf16."""
    n = mpk_rmsnorm(x, w, eps).float()
    d = x.shape[-1]
    c, s = cos.float(), sin.float()
    lo, hi = n[..., : d // 2], n[..., d // 2:]
    out = torch.cat((lo * c[..., : d // 2] - hi * s[..., : d // 2],
                     hi * c[..., d // 2:] + lo * s[..., d // 2:]), dim=-1)
    return out.to(BF16)


def mpk_attention_decode(q, k, v):
    """One query token: q [n_q, d] bf16, k/v [L, n_kv, d] bf16 (already holding
    the new token).  Softmax scale 1/sqrt(d) (attention_sm100.cuh:85), fp32
    softmax and accumulation, bf16 output."""
    n_q, d = q.shape
    n_kv = k.shape[1]
    rep = n_q // n_kv
    kf = k.float().repeat_interleave(rep, dim=1)  # [L, n_q, d]
    vf = v.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("hd,lhd->hl", q.float(), kf) / math.sqrt(d)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hl,lhd->hd", p, vf).to(BF16)


def mpk_argmax(logits):
    """Greedy token over bf16 logits; ties go to the lowest index (torch's rule,
    demo/qwen3/demo.py:1207)."""
    return logits.float().argmax(-1)


class MpkRefModel:
    """The decode path with the megakernel's task arithmetic, one token per
    request per iteration (prompt tokens are fed through the same path)."""

    def __init__(self, geom: Geometry, weights: dict, max_seq: int, layers: int | None = None):
        self.g, self.w = geom, weights
        self.n_layers = geom.layers if layers is None else layers
        self.k_cache = torch.zeros(self.n_layers, max_seq, geom.n_kv, geom.head_dim, dtype=BF16)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.cos, self.sin = rope_tables(geom, max_seq)

    def qkv_weight(self, i):
        w = self.w
        return torch.cat((w[f"l{i}.q"], w[f"l{i}.k"], w[f"l{i}.v"]), 0)

    @torch.inference_mode()
    def layer(self, i, x, pos):
        """x [hidden] bf16 at position pos -> [hidden] bf16."""
        g, w = self.g, self.w
        d = g.head_dim
        xn = mpk_rmsnorm(x, w[f"l{i}.ln1"], g.eps)
        qkv = mpk_linear(xn, self.qkv_weight(i))
        q = qkv[: g.n_q * d].view(g.n_q, d)
        k = qkv[g.n_q * d: (g.n_q + g.n_kv) * d].view(g.n_kv, d)
        v = qkv[(g.n_q + g.n_kv) * d:].view(g.n_kv, d)
        q = mpk_qk_norm_rope(q, w[f"l{i}.qn"], self.cos[pos], self.sin[pos], g.eps)
        k = mpk_qk_norm_rope(k, w[f"l{i}.kn"], self.cos[pos], self.sin[pos], g.eps)
        self.k_cache[i, pos] = k
        self.v_cache[i, pos] = v
        a = mpk_attention_decode(q, self.k_cache[i, : pos + 1], self.v_cache[i, : pos + 1]).reshape(-1)
        x = mpk_linear(a, w[f"l{i}.o"], residual=x)
        xn = mpk_rmsnorm(x, w[f"l{i}.ln2"], g.eps)
        h = mpk_silu_mul(mpk_linear(xn, w[f"l{i}.gate"]), mpk_linear(xn, w[f"l{i}.up"]))
        return mpk_linear(h, w[f"l{i}.down"], residual=x)

    @torch.inference_mode()
    def step(self, token, pos):
        x = self.w["embed"][token]
        for i in range(self.n_layers):
            x = self.layer(i, x, pos)
        xn = mpk_rmsnorm(x, self.w["norm"], self.g.eps)
        return mpk_linear(xn, self.w["lm_head"])

    @torch.inference_mode()
    def generate(self, prompt, n_new):
        toks = prompt.tolist()
        P = len(toks)
        logits_out = []
        for p in range(P + n_new - 1):
            lg = self.step(toks[p], p)
            if p >= P - 1:
                logits_out.append(lg.clone())
                toks.append(int(mpk_argmax(lg)))
        return toks, torch.stack(logits_out)


# ---------------------------------------------------------------------------
# comparators
# ---------------------------------------------------------------------------
def max_rel_err(a, b):
    """Max |a-b| normalised by the largest |b| of the row: relative error on
    logits near zero is ill-posed, so the step's logit scale is the unit."""
    a, b = a.float(), b.float()
    scale = b.abs().amax(-1, keepdim=True).clamp_min(1e-30)
    return float(((a - b).abs() / scale).max())


def top2_margin(logits):
    t = logits.float().topk(2, dim=-1).values
    return t[..., 0] - t[..., 1]


# ---------------------------------------------------------------------------
# Qwen3-MoE (the reference's MoE demo, demo/qwen3/demo_30B_A3B.py)
# ---------------------------------------------------------------------------
# The PyTorch side of that demo is transformers' Qwen3MoeForCausalLM (demo_30B_A3B.py:1, 381-392), a
# third-party dependency whose source is not part of the reference tree (pinned transformers==4.57.1 in
# requirements.txt; this image has 5.5.0).  TorchMoeRefModel restates its published algorithm
# (models/qwen3_moe/modeling_qwen3_moe.py of transformers: Qwen3MoeRMSNorm, Qwen3MoeAttention with the default
# sdpa attention, Qwen3MoeTopKRouter, Qwen3MoeExperts, Qwen3MoeSparseMoeBlock, Qwen3MoeDecoderLayer) and is
# pinned by tests/golden/make_golden_moe.py, which runs the installed transformers model on the same seeded
# weights and commits ITS outputs as the fixture.
@dataclass(frozen=True)
class MoeGeometry:
    hidden: int = 2048
    n_q: int = 32
    n_kv: int = 4
    head_dim: int = 128
    experts: int = 128
    top_k: int = 8
    moe_mlp: int = 768
    layers: int = 48
    vocab: int = 151936
    rope_theta: float = 1e6
    eps: float = 1e-6
    init_std: float = 0.02

    def asdict(self):
        return asdict(self)


QWEN3_30B_A3B = MoeGeometry()
MOE_TINY = MoeGeometry(hidden=512, n_q=8, n_kv=2, experts=16, top_k=4, moe_mlp=256, layers=2, vocab=2048)


def moe_weight_names(g: MoeGeometry):
    names = [("embed", (g.vocab, g.hidden))]
    for i in range(g.layers):
        names += [(f"l{i}.q", (g.n_q * g.head_dim, g.hidden)), (f"l{i}.k", (g.n_kv * g.head_dim, g.hidden)),
                  (f"l{i}.v", (g.n_kv * g.head_dim, g.hidden)), (f"l{i}.o", (g.hidden, g.n_q * g.head_dim)),
                  (f"l{i}.router", (g.experts, g.hidden)), (f"l{i}.w13", (g.experts, 2 * g.moe_mlp, g.hidden)),
                  (f"l{i}.w2", (g.experts, g.hidden, g.moe_mlp))]
    names.append(("lm_head", (g.vocab, g.hidden)))
    return names


def make_moe_weights(g: MoeGeometry, seed: int = 0, device: str = "cpu", norm_jitter: float = 0.0, router_std: float = 2.0):
    """bf16 weights ~ N(0, init_std) in the order of ``moe_weight_names``; the router rows are scaled by
    ``router_std / init_std`` so that the routing logits spread (with N(0, 0.02) rows every expert scores the
    same to within bf16 noise and the top-k would be decided by rounding)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in moe_weight_names(g):
        t = torch.randn(shape, generator=gen, dtype=torch.float32, device=device)
        std = router_std / math.sqrt(g.hidden) if name.endswith(".router") else g.init_std
        w[name] = (t * std).to(BF16)
        del t

    def norm(n):
        if norm_jitter == 0.0:
            return torch.ones(n, dtype=BF16, device=device)
        u = torch.rand(n, generator=gen, dtype=torch.float32, device=device)
        return (1.0 + norm_jitter * (2 * u - 1)).to(BF16)

    for i in range(g.layers):
        w[f"l{i}.ln1"], w[f"l{i}.ln2"] = norm(g.hidden), norm(g.hidden)
        w[f"l{i}.qn"], w[f"l{i}.kn"] = norm(g.head_dim), norm(g.head_dim)
    w["norm"] = norm(g.hidden)
    return w


def hf_rmsnorm(x, w, eps=1e-6):
    """Qwen3MoeRMSNorm.forward: fp32 normalisation with eps, cast back, then the weight."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return w * xf.to(x.dtype)


def moe_route(logits, top_k):
    """Qwen3MoeTopKRouter.forward (norm_topk_prob=True): fp32 softmax over the experts, top-k, renormalised."""
    p = torch.softmax(logits, dtype=torch.float, dim=-1)
    val, idx = torch.topk(p, top_k, dim=-1)
    val = val / val.sum(dim=-1, keepdim=True)
    return val, idx


class TorchMoeRefModel:
    """Batch-1 restatement of transformers' Qwen3MoeForCausalLM (sdpa attention) with a contiguous KV cache."""

    def __init__(self, g: MoeGeometry, weights: dict, max_seq: int, layers: int | None = None, device: str = "cpu"):
        self.g, self.w, self.device = g, weights, device
        self.n_layers = g.layers if layers is None else layers
        self.k_cache = torch.zeros(self.n_layers, g.n_kv, max_seq, g.head_dim, dtype=BF16, device=device)
        self.v_cache = torch.zeros_like(self.k_cache)
        d = g.head_dim
        inv_freq = 1.0 / (g.rope_theta ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        freqs = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        self.cos, self.sin = emb.cos().to(BF16).to(device), emb.sin().to(BF16).to(device)

    def _attention(self, i, h, pos0):
        g, w = self.g, self.w
        n = h.shape[0]
        x = hf_rmsnorm(h, w[f"l{i}.ln1"], g.eps)
        q = hf_rmsnorm(F.linear(x, w[f"l{i}.q"]).view(n, g.n_q, g.head_dim), w[f"l{i}.qn"], g.eps).transpose(0, 1)
        k = hf_rmsnorm(F.linear(x, w[f"l{i}.k"]).view(n, g.n_kv, g.head_dim), w[f"l{i}.kn"], g.eps).transpose(0, 1)
        v = F.linear(x, w[f"l{i}.v"]).view(n, g.n_kv, g.head_dim).transpose(0, 1)
        cos, sin = self.cos[pos0:pos0 + n][None], self.sin[pos0:pos0 + n][None]
        q = (q * cos) + (ref_rotate_half(q) * sin)
        k = (k * cos) + (ref_rotate_half(k) * sin)
        self.k_cache[i, :, pos0:pos0 + n] = k
        self.v_cache[i, :, pos0:pos0 + n] = v
        L = pos0 + n
        # sdpa_attention_forward of transformers: torch's scaled_dot_product_attention, causal for a multi-token prefill
        o = F.scaled_dot_product_attention(q[None], self.k_cache[i, :, :L][None], self.v_cache[i, :, :L][None],
                                           is_causal=(n > 1), enable_gqa=True)[0]
        o = o.transpose(0, 1).reshape(n, g.n_q * g.head_dim)
        return F.linear(o, w[f"l{i}.o"])

    def _moe(self, i, h):
        g, w = self.g, self.w
        x = hf_rmsnorm(h, w[f"l{i}.ln2"], g.eps)
        router_logits = F.linear(x, w[f"l{i}.router"])
        val, idx = moe_route(router_logits, g.top_k)
        # how decisively the last token's top-k set was chosen: the gap between the k-th and the (k+1)-th logit
        top = router_logits[-1].float().topk(g.top_k + 1).values
        self.route_margin = min(self.route_margin, float(top[g.top_k - 1] - top[g.top_k]))
        out = torch.zeros_like(x)
        for e in sorted(set(idx.flatten().tolist())):  # Qwen3MoeExperts.forward: experts in index order
            slot, tok = torch.where((idx == e).t())
            cur = x[tok]
            gate, up = F.linear(cur, w[f"l{i}.w13"][e]).chunk(2, dim=-1)
            cur = F.linear(F.silu(gate) * up, w[f"l{i}.w2"][e])
            cur = cur * val[tok, slot, None]
            out.index_add_(0, tok, cur.to(out.dtype))
        return out

    @torch.inference_mode()
    def forward(self, token_ids, pos0):
        """Logits of the given tokens; ``self.route_margin`` is left at the smallest routing gap, over the layers,
        of the LAST token (a small gap means another arithmetic may pick a different expert set there)."""
        h = F.embedding(token_ids.to(self.device), self.w["embed"])
        self.route_margin = float("inf")
        for i in range(self.n_layers):
            h = h + self._attention(i, h, pos0)
            h = h + self._moe(i, h)
        return F.linear(hf_rmsnorm(h, self.w["norm"], self.g.eps), self.w["lm_head"])

    @torch.inference_mode()
    def generate(self, prompt, n_new, forced=None):
        toks = prompt.clone().tolist()
        P = len(toks)
        logits_out, self.margins = [], []
        lg = self.forward(torch.tensor(toks), 0)
        for j in range(n_new):
            last = lg[-1]
            logits_out.append(last.clone().cpu())
            self.margins.append(self.route_margin)
            toks.append(int(last.argmax(-1)) if forced is None else int(forced[j]))
            if j + 1 < n_new:
                lg = self.forward(torch.tensor([toks[-1]]), P + j)
        return toks, torch.stack(logits_out)
