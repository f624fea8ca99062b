"""Plain, slow restatement of the Nafazen design: one function per mechanism, whole sequences only, no cache, no
paging, no batching.  It is the oracle of the Nafazen tests and shares no code with the framework's model, ops or
kernels.  Everything runs in float32 on the CPU (``exact=True``), or with matrix products on bfloat16-rounded
operands (``exact=False``) to mimic the serving precision.

Notation: T tokens, W model width, H heads, dn / dr unrotated / rotated query-key sizes per head, dv value size,
R latent size.  Weights are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def _mm(x: torch.Tensor, w: torch.Tensor, exact: bool) -> torch.Tensor:
    if exact:
        return x.float() @ w.float().t()
    return (x.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().t())


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is a single number."""
    return rms(x, eps) * float(g)


def vector_norm(x, w, eps):
    return rms(x, eps) * w.float()


def rotary_frequencies(rot: Dict) -> (torch.Tensor, float):
    """Per-pair frequencies and the factor on cos / sin (1 without scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    mult = 1.0
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / factor * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.float(), mult


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, rot: Dict) -> torch.Tensor:
    """x: [T, ..., n] with n >= rot.dims; pairs (2i, 2i+1) of the first rot.dims coordinates are rotated."""
    dims = int(rot["dims"])
    f, mult = rotary_frequencies(rot)
    ang = positions.float().unsqueeze(-1) * f                      # [T, dims/2], float32
    cos, sin = torch.cos(ang) * mult, torch.sin(ang) * mult
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    x = x.float()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_kv(h, p: Dict[str, torch.Tensor], mx: Dict, positions, eps, exact):
    """The cached pair of a latent-attention layer: normed latent [T, R] and rotated shared key part [T, dr]."""
    R = int(mx["kv_rank"])
    d = _mm(h, p["dkv"], exact)
    c = vector_norm(d[:, :R], p["dkv.norm"], eps)
    kr = rotate_interleaved(d[:, R:], positions, mx["rot"])
    return c, kr


def latent_attention(h, p: Dict[str, torch.Tensor], mx: Dict, positions, eps, exact, shared_kv=None):
    """Causal latent attention over one whole sequence.  ``shared_kv`` = (c, kr) of another layer, for a layer
    that has no down-projection of its own."""
    T = h.shape[0]
    H, dn, dr, dv = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"])
    cq = vector_norm(_mm(h, p["dq"], exact), p["dq.norm"], eps)
    q = _mm(cq, p["uq"], exact).view(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate_interleaved(q[..., dn:], positions, mx["rot"])
    c, kr = shared_kv if shared_kv is not None else latent_kv(h, p, mx, positions, eps, exact)
    kn = _mm(c, p["uk"], exact).view(T, H, dn)
    v = _mm(c, p["uv"], exact).view(T, H, dv)
    if not exact:
        qn, qr, kn, kr_, v = (t.to(torch.bfloat16).float() for t in (qn, qr, kn, kr, v))
    else:
        kr_ = kr
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr_)) * float(mx["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    w = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * dv)
    return _mm(o, p["o"], exact), (c, kr)


def xielu(z, pq):
    z = z.float()
    a_p = torch.nn.functional.softplus(pq[0].float())
    a_n = 0.5 + torch.nn.functional.softplus(pq[1].float())
    return torch.where(z > 0, a_p * z * z + 0.5 * z, a_n * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense_ff(h, p, exact):
    return _mm(xielu(_mm(h, p["up"], exact), p["act"]), p["down"], exact)


def gated_expert(h, p, prefix, exact):
    g = _mm(h, p[prefix + "gate"], exact)
    u = _mm(h, p[prefix + "up"], exact)
    return _mm(torch.nn.functional.silu(g) * u, p[prefix + "down"], exact)


def route(h, w_router, top: int):
    """sigmoid scores of the chosen experts (largest first) and their indices; not renormalised."""
    s = torch.sigmoid(h.float() @ w_router.float().t())
    val, idx = torch.topk(s, top, dim=-1)
    return val, idx


def moe_ff(h, p, mlp: Dict, exact):
    T = h.shape[0]
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    hin = h.float() if exact else h.to(torch.bfloat16).float()
    val, idx = route(hin, p["router"], top)
    out = torch.zeros(T, p["e0.down"].shape[0])
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += gated_expert((val[t, k] * h[t].float()).unsqueeze(0), p, f"e{e}.", exact)[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(hin @ p["shared.sg"].float().t())          # [T, 1]
        out = out + gate * gated_expert(h, p, "shared.", exact)
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens: List[int], exact: bool = True,
            trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``trace`` collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    pos = torch.arange(len(tokens))
    x = weights["embed"].float()[torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    kv: Dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        mx, p = layer["mixer"], sub(weights, f"l{i}.mix.")
        if layer["type"] not in ("latent_attention", "latent_attention_2"):
            raise ValueError(layer["type"])
        src = mx.get("kv_from")
        y, kv[i] = latent_attention(x, p, mx, pos, eps, exact, shared_kv=None if src is None else kv[int(src)])
        x = x + scalar_norm(y, weights[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            q = sub(weights, f"l{i}.mlp.")
            y = dense_ff(x, q, exact) if mlp["kind"] == "dense" else moe_ff(x, q, mlp, exact)
            x = x + scalar_norm(y, weights[f"l{i}.norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    y = scalar_norm(x, weights["final.norm"], eps)
    logits = _mm(y, weights["head"], exact)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


def random_weights(cfg: Dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights in the layout the design's checkpoints use."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])
    out: Dict[str, torch.Tensor] = {}

    def lin(name, o, i, gain=1.0):
        out[name] = (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).to(dtype)

    lin("embed", int(cfg["vocab"]), W, math.sqrt(W))
    for i, layer in enumerate(cfg["layers"]):
        mx, pre = layer["mixer"], f"l{i}."
        H, dn, dr, dv, R, Q = (int(mx[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
        out[pre + "norm1"] = (0.5 + torch.rand((), generator=g)).to(dtype)
        lin(pre + "mix.dq", Q, W)
        out[pre + "mix.dq.norm"] = (0.5 + torch.rand(Q, generator=g)).to(dtype)
        lin(pre + "mix.uq", H * (dn + dr), Q, 2.0)
        if mx.get("kv_from") is None:
            lin(pre + "mix.dkv", R + dr, W)
            out[pre + "mix.dkv.norm"] = (0.5 + torch.rand(R, generator=g)).to(dtype)
        lin(pre + "mix.uk", H * dn, R, 2.0)
        lin(pre + "mix.uv", H * dv, R)
        lin(pre + "mix.o", W, H * dv)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[pre + "norm2"] = (0.5 + torch.rand((), generator=g)).to(dtype)
        if mlp["kind"] == "dense":
            lin(pre + "mlp.up", int(mlp["ff"]), W)
            lin(pre + "mlp.down", W, int(mlp["ff"]))
            out[pre + "mlp.act"] = torch.randn(2, generator=g).to(dtype)
        else:
            ff = int(mlp["expert"]["ff"])
            for e in range(int(mlp["router"]["experts"])):
                lin(pre + f"mlp.e{e}.gate", ff, W)
                lin(pre + f"mlp.e{e}.up", ff, W)
                lin(pre + f"mlp.e{e}.down", W, ff)
            lin(pre + "mlp.router", int(mlp["router"]["experts"]), W, 2.0)
            if mlp.get("shared") is not None:
                sf = int(mlp["shared"]["ff"])
                lin(pre + "mlp.shared.gate", sf, W)
                lin(pre + "mlp.shared.up", sf, W)
                lin(pre + "mlp.shared.down", W, sf)
                lin(pre + "mlp.shared.sg", 1, W)
    out["final.norm"] = (0.5 + torch.rand((), generator=g)).to(dtype)
    lin("head", int(cfg["vocab"]), W)
    return out
