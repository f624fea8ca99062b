"""A plain, slow restatement of the Teluzen design for tests: one function per mechanism, whole sequences at once, no
cache, no batching, float64 throughout.  It shares no code with the package.

Notation: T tokens, W width, H query heads, G key/value heads, d query/key size, e value size, S window size, P pool
size.  ``tensors`` maps checkpoint names to torch tensors; ``cfg`` is the parsed config.json dictionary."""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotary_spectrum(dims: int, base: float, scaling: Optional[dict]):
    """Frequencies of the dims/2 rotated pairs and the amplitude of cos and sin."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    amp = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def where(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        out = []
        for i, fi in enumerate(f):
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / factor * r + fi * (1 - r))
        f = out
        amp = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=F64), amp


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """x: [T, heads, d]; the first ``dims`` numbers of every head are rotated as pairs (2i, 2i+1)."""
    f, amp = rotary_spectrum(dims, base, scaling)
    a = positions.to(F64)[:, None] * f[None, :]                      # [T, dims/2]
    c, s = (torch.cos(a) * amp)[:, None, :], (torch.sin(a) * amp)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def pooled(k: torch.Tensor, P: int) -> torch.Tensor:
    """Means of the complete blocks of P consecutive rows of k [T, ...] -> [T // P, ...]."""
    n = k.shape[0] // P
    return k[:n * P].reshape(n, P, *k.shape[1:]).mean(1)


def visibility(T: int, S: Optional[int], P: Optional[int]):
    """(token mask [T, T], block mask [T, T // P]): query i sees token j iff 0 <= i - j < S, and block b iff its last
    position b P + P - 1 <= i - S."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    if S is None:
        return (j <= i), torch.zeros(T, 0, dtype=torch.bool)
    tok = (j <= i) & (i - j < S)
    nb = T // P
    b = torch.arange(nb)[None, :]
    blk = (b * P + P - 1) <= (i - S)
    return tok, blk


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, m: dict, t: Dict[str, torch.Tensor], pre: str, eps: float,
                    v_first: Optional[torch.Tensor], cache_round: Callable = lambda z: z):
    """h: [T, W].  Returns (output [T, W], the values this layer caches [T, G, e], its own unmixed values)."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ t[pre + "q"].T + t[pre + "q.b"]
    k = h @ t[pre + "k"].T + t[pre + "k.b"]
    v = h @ t[pre + "v"].T + t[pre + "v.b"]
    q = rms_norm(q, t[pre + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, t[pre + "k.norm"], eps).reshape(T, G, d)
    v = v.reshape(T, G, e)
    rot = m.get("rot")
    if rot:
        q = rotate_pairs(q, positions, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_pairs(k, positions, rot["dims"], rot["base"], rot.get("scaling"))
    v_own = v
    if m.get("v_mix") and v_first is not None:
        lam = t[pre + "vmix"].reshape(())
        v = (1 - lam) * v + lam * v_first
    mask = m.get("mask")
    S, P = (mask["size"], mask["pool"]) if mask else (None, None)
    o = attend(q, cache_round(k), cache_round(v), S, P, m["scale"], t[pre + "temp"], t[pre + "talk"], cache_round)
    return o.reshape(T, H * e) @ t[pre + "o"].T, v, v_own


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, S: Optional[int], P: Optional[int], scale: float,
           temp: Optional[torch.Tensor], talk: Optional[torch.Tensor], cache_round: Callable = lambda z: z) -> torch.Tensor:
    """q: [T, H, d], k: [T, G, d], v: [T, G, e] of one sequence from position 0 -> [T, H, e]."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    tok, blk = visibility(T, S, P)
    keys, vals, vis = k, v, tok
    if S is not None and T // P > 0:
        keys = torch.cat([cache_round(pooled(k, P)), k], 0)
        vals = torch.cat([cache_round(pooled(v, P)), v], 0)
        vis = torch.cat([blk, tok], 1)
    kh = keys.repeat_interleave(rep, dim=1)                                  # [N, H, d]
    s = torch.einsum("thd,nhd->htn", q, kh) * scale
    if temp is not None:
        s = s * temp[:, None, None]
    s = s.masked_fill(~vis[None], float("-inf"))
    w = torch.softmax(s, -1)
    if talk is not None:
        w = torch.einsum("hg,gtn->htn", talk, w)
    vh = vals.repeat_interleave(rep, dim=1)                                  # [N, H, e]
    return torch.einsum("htn,nhe->the", w, vh)


def dense_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    z = torch.relu(h @ t[pre + "up"].T)
    return (z * z) @ t[pre + "down"].T


def gated_expert(h: torch.Tensor, t: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    g = h @ t[pre + "gate"].T
    return ((g * torch.sigmoid(g)) * (h @ t[pre + "up"].T)) @ t[pre + "down"].T


def route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    z = h @ w_router.T
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def moe_ff(h: torch.Tensor, mlp: dict, t: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    idx, wt = route(h, t[pre + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for r in range(h.shape[0]):
        for c in range(idx.shape[1]):
            out[r] += wt[r, c] * gated_expert(h[r:r + 1], t, f"{pre}e{int(idx[r, c])}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, t, pre + "shared.")
    return out


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], cache_round: Callable = lambda z: z):
    """Returns (logits [T, vocab], [residual stream after every layer])."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = t["embed"][torch.tensor(tokens)] + t["pos"][pos]
    v_first = None
    trace = []
    for i, layer in enumerate(cfg["layers"]):
        assert layer["type"] == "attention"
        p = f"l{i}."
        y, _, v_own = attention_mixer(rms_norm(x, t[p + "norm1"], eps), pos, layer["mixer"], t, p + "mix.", eps, v_first, cache_round)
        if layer["mixer"].get("v_mix") and v_first is None:
            v_first = v_own
        x = x + rms_norm(y, t[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, t[p + "norm2"], eps)
            y = dense_ff(h, t, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, mlp, t, p + "mlp.")
            x = x + rms_norm(y, t[p + "norm2b"], eps)
        trace.append(x.clone())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T, trace


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors under the checkpoint names, fp32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    t: Dict[str, torch.Tensor] = {}

    def mat(name, out, inp, gain=1.0):
        t[name] = torch.randn(out, inp, generator=g) * gain / inp ** 0.5

    def vec(name, n, mean=1.0, std=0.2):
        t[name] = mean + std * torch.randn(n, generator=g)
    t["embed"] = torch.randn(cfg["vocab"], W, generator=g)
    t["pos"] = 0.5 * torch.randn(cfg["max_positions"], W, generator=g)
    mat("head", cfg["vocab"], W)
    vec("final.norm", W)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm1b"):
            vec(p + n, W)
        mat(p + "mix.q", H * d, W, 2.0)
        mat(p + "mix.k", G * d, W, 2.0)
        mat(p + "mix.v", G * e, W)
        vec(p + "mix.q.b", H * d, 0.0, 0.3)
        vec(p + "mix.k.b", G * d, 0.0, 0.3)
        vec(p + "mix.v.b", G * e, 0.0, 0.3)
        vec(p + "mix.q.norm", H * d)
        vec(p + "mix.k.norm", G * d)
        vec(p + "mix.temp", H, 1.0, 0.3)
        t[p + "mix.talk"] = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
        t[p + "mix.vmix"] = torch.tensor(0.35) + 0.1 * torch.randn((), generator=g)
        mat(p + "mix.o", W, H * e)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        for n in ("norm2", "norm2b"):
            vec(p + n, W)
        if mlp["kind"] == "dense":
            mat(p + "mlp.up", mlp["ff"], W)
            mat(p + "mlp.down", W, mlp["ff"])
            continue
        names = [f"e{k}." for k in range(mlp["router"]["experts"])] + (["shared."] if mlp.get("shared") else [])
        for n in names:
            ff = mlp["shared"]["ff"] if n == "shared." else mlp["expert"]["ff"]
            mat(p + "mlp." + n + "gate", ff, W)
            mat(p + "mlp." + n + "up", ff, W)
            mat(p + "mlp." + n + "down", W, ff)
        mat(p + "mlp.router", mlp["router"]["experts"], W, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in t.items()}
