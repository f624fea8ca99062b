"""Teluzen: a decoder-only design of pooled-window attention mixers (``models/mixers.py``) and squared-ReLU or
mixture-of-experts feed-forwards (``models/ffn.py``) in a sandwich-norm residual layout:

    x <- x + n1b(mixer(n1(x)));   x <- x + n2b(ff(n2(x)))          n(v) = w * v / sqrt(mean(v^2) + eps)

The residual stream ``x`` is fp32 and starts as ``embed[token] + pos[position]`` (learned absolute positions); the
output is ``head(final_norm(x))``.  The mixer is grouped-query attention with projection biases, an RMS norm over the
whole q and k projections, partial interleaved rotation (YaRN-blended spectrum when the configuration has ``scaling``),
a score temperature per head, a sliding window plus mean-pooled blocks before it, mixing of the softmax weights across
heads, and value mixing with the first ``v_mix`` layer.  Experts are gated-SiLU; the ``top`` largest router logits are
chosen and weighted by a softmax over the chosen logits; a shared expert is added for every token.  The layer list,
every size and every constant come from the checkpoint's ``config.json``:

    {"architecture": "Teluzen", "width", "vocab", "max_positions", "norm": {"eps"},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "v_mix", "mask": {"size", "pool"},
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}?}},
                 "mlp": null | {"kind": "dense", "ff"} |
                        {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"}?}}, ...]}

Checkpoint tensors: ``embed``, ``pos``, ``head``, ``final.norm``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.{q,k,v}`` with ``.b`` biases, ``l<i>.mix.{q.norm,k.norm,temp,talk,vmix,o}``, ``l<i>.mlp.{up,down}`` or
``l<i>.mlp.{router,e<k>.{gate,up,down},shared.{gate,up,down}}``; linear weights are [out, in].  The model runs ragged
paged batches only (``forward_ragged``); the serving engine owns the caches.

Reference: none — the reference serves whatever HF returns (reference llmctl/serve/server.py:127-160)."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import elementwise as eops
from ..ops import functional as ops
from .ffn import GatedExpertMoE, SquaredReluMLP
from .mixers import PooledWindowAttention, PooledWindowAttentionSpec
from .registry import Architecture, register_architecture

MIXER_TYPES = ("attention",)


@dataclass
class TeluzenLayer:
    type: str
    mixer: PooledWindowAttentionSpec
    mlp: Optional[Dict[str, Any]]


@dataclass
class TeluzenConfig:
    name: str = "teluzen"
    width: int = 256
    vocab_size: int = 512
    max_position_embeddings: int = 2048       # rows of the learned position table
    norm_eps: float = 1e-5
    layers: List[TeluzenLayer] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], name: str = "teluzen") -> "TeluzenConfig":
        layers: List[TeluzenLayer] = []
        first_mix: Optional[PooledWindowAttentionSpec] = None
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r} (known: {MIXER_TYPES})")
            m = l["mixer"]
            rot = m.get("rot") or {}
            mask = m.get("mask") or {}
            spec = PooledWindowAttentionSpec(
                heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                scale=float(m["scale"]), window=int(mask.get("size", 0)), pool=int(mask.get("pool", 0)),
                rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)), rot_scaling=rot.get("scaling") or None,
                bias=True, qk_norm=True, head_temperature=True, talking_heads=True, v_mix=bool(m.get("v_mix", False)))
            if spec.heads % spec.kv_heads:
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if spec.window and spec.pool < 1:
                raise ValueError(f"layer {i}: a window needs a pool size of at least 1")
            if spec.v_mix:
                if first_mix is None:
                    first_mix = spec
                elif (first_mix.kv_heads, first_mix.vdim) != (spec.kv_heads, spec.vdim):
                    raise ValueError(f"layer {i}: value mixing needs the value sizes of the first v_mix layer")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(TeluzenLayer(l["type"], spec, mlp))
        return cls(name=name, width=int(d["width"]), vocab_size=int(d["vocab"]), max_position_embeddings=int(d["max_positions"]),
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)), layers=layers, raw=d)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def num_parameters(self) -> int:
        with torch.device("meta"):
            m = TeluzenModel(self, dtype=torch.bfloat16, device="meta")
        return sum(p.numel() for p in m.parameters())


class TeluzenBlock(nn.Module):
    def __init__(self, cfg: TeluzenConfig, layer: TeluzenLayer, dtype, device):
        super().__init__()
        W = cfg.width

        def norm_weight():
            return nn.Parameter(torch.ones(W, dtype=torch.float32, device=device))
        self.mixer = PooledWindowAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        self.norm1, self.norm1b = norm_weight(), norm_weight()
        mlp = layer.mlp
        self.mlp: Optional[nn.Module] = None
        if mlp is not None:
            self.norm2, self.norm2b = norm_weight(), norm_weight()
            if mlp["kind"] == "dense":
                self.mlp = SquaredReluMLP(W, int(mlp["ff"]), dtype, device)
            else:
                shared = mlp.get("shared")
                self.mlp = GatedExpertMoE(W, int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]),
                                          int(shared["ff"]) if shared else None, dtype, device, scale_input=False,
                                          softmax_scores=2, renormalise=False, shared_gate=False)


class TeluzenModel(nn.Module):
    ragged = True           # runs ragged paged batches through ``forward_ragged`` (serve/engine.py)

    def __init__(self, cfg: TeluzenConfig, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))
        self.pos = nn.Parameter(torch.empty(cfg.max_position_embeddings, cfg.width, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([TeluzenBlock(cfg, l, dtype, device) for l in cfg.layers])
        self.final_norm = nn.Parameter(torch.ones(cfg.width, dtype=torch.float32, device=device))
        self.head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))

    # ---- weights ---------------------------------------------------------------------------------------
    def load_state(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint names -> tensors (any float type; converted to the model's)."""
        dev = self.embed.device

        def get(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            return tensors[name].to(dev)
        with torch.no_grad():
            self.embed.copy_(get("embed"))
            self.pos.copy_(get("pos"))
            self.head.copy_(get("head"))
            self.final_norm.copy_(get("final.norm").float())
            for i, blk in enumerate(self.blocks):
                blk.norm1.copy_(get(f"l{i}.norm1").float())
                blk.norm1b.copy_(get(f"l{i}.norm1b").float())
                blk.mixer.load(get, f"l{i}.mix.")
                if blk.mlp is not None:
                    blk.norm2.copy_(get(f"l{i}.norm2").float())
                    blk.norm2b.copy_(get(f"l{i}.norm2b").float())
                    blk.mlp.load(get, f"l{i}.mlp.")

    def init_random(self, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                leaf = name.rsplit(".", 1)[-1]
                if leaf == "talk":
                    p.copy_(torch.eye(p.shape[0]) + 0.2 * torch.randn(p.shape, generator=g))
                elif leaf == "vmix":
                    p.fill_(0.3)
                elif leaf == "b_qkv":
                    p.copy_((0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
                elif leaf == "pos":
                    p.copy_((0.5 * torch.randn(p.shape, generator=g)).to(p.dtype))
                elif p.dim() == 1:
                    p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
                else:
                    p.copy_((torch.randn(p.shape, generator=g) / p.shape[-1] ** 0.5).to(p.dtype))

    # ---- caches ----------------------------------------------------------------------------------------
    def cache_bytes_per_block(self, block_size: int) -> int:
        it = torch.empty((), dtype=self.dtype).element_size()
        return sum(l.mixer.rows_per_page(block_size) * l.mixer.cache_width for l in self.cfg.layers) * it

    def allocate_caches(self, num_blocks: int, block_size: int, device) -> List[torch.Tensor]:
        """One ``[pages, block_size + pooled rows, G (d + e)]`` tensor per layer: the token rows ``[keys | values]`` of a
        page and, behind them, the pooled rows of the blocks that start in it."""
        return [torch.zeros(num_blocks, l.mixer.rows_per_page(block_size), l.mixer.cache_width, dtype=self.dtype, device=device)
                for l in self.cfg.layers]

    # ---- forward ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_ragged(self, batch, caches: List[torch.Tensor], layer_trace: Optional[list] = None) -> torch.Tensor:
        """``batch``: serve.ragged.RaggedBatch.  Returns fp32 logits [len(batch.out_rows), vocab]."""
        cfg, dt, eps = self.cfg, self.dtype, self.cfg.norm_eps
        blocks = self.blocks
        x = eops.embed_positions(batch.tokens, batch.positions, self.embed, self.pos)
        h = eops.rmsnorm_rows(x, None, blocks[0].norm1, eps, dt) if len(blocks) else None
        v_first = None
        for i, blk in enumerate(blocks):
            after = blocks[i + 1].norm1 if i + 1 < len(blocks) else None        # in-norm of the sublayer that follows
            y, v_first = blk.mixer(h, batch, caches[i], v_first)
            if blk.mlp is None:
                h = eops.sandwich_residual(y, x, blk.norm1b, after, eps, dt)
            else:
                # the feed-forward's input in the activation type and unrounded (the router of a mixture reads the latter)
                if isinstance(blk.mlp, GatedExpertMoE):
                    h, h32 = eops.sandwich_residual(y, x, blk.norm1b, blk.norm2, eps, dt, want_fp32=True)
                else:
                    h = h32 = eops.sandwich_residual(y, x, blk.norm1b, blk.norm2, eps, dt)
                y = blk.mlp(h, h32)
                h = eops.sandwich_residual(y, x, blk.norm2b, after, eps, dt)
            if layer_trace is not None:
                layer_trace.append(x.clone())
        if batch.num_out == 0:                  # a step that only fills the caches
            return torch.empty(0, cfg.vocab_size, dtype=torch.float32, device=x.device)
        y = eops.rmsnorm_rows(x, batch.out_rows, self.final_norm, eps, dt)
        if y.is_cuda and dt == torch.bfloat16 and ops.kernel_config().gemm == "native" and ops._gemm_ok(y, self.head) \
                and self.head.shape[0] % 8 == 0:
            return ops.gemm_raw(y, self.head, out_dtype=torch.float32)
        return torch.nn.functional.linear(y, self.head).float()


def _load_weights(model: TeluzenModel, directory) -> None:
    from safetensors.torch import load_file
    model.load_state(load_file(str(Path(directory) / "model.safetensors")))


def build_teluzen(cfg: TeluzenConfig, *, dtype=torch.bfloat16, device=None, seed: int = 42, **_ignored) -> TeluzenModel:
    m = TeluzenModel(cfg, dtype=dtype, device=device)
    m.init_random(seed)
    return m


register_architecture(Architecture(name="Teluzen", config_from_dict=TeluzenConfig.from_dict, config_type=TeluzenConfig,
                                   build=build_teluzen, load_weights=_load_weights))


def example_config(width: int = 48, vocab: int = 80, heads: int = 4, kv_heads: int = 2, dim: int = 8, vdim: int = 6,
                   rot_dims: int = 4, window: int = 12, pool: int = 4, ff: int = 40, experts: int = 5, top: int = 2,
                   expert_ff: int = 16, shared_ff: Optional[int] = 24, pattern: str = "DMMD", v_mix: str = "0110",
                   yarn: bool = True, max_positions: int = 512, scale: Optional[float] = None) -> Dict[str, Any]:
    """A small configuration dictionary for tests, benchmarks and examples.  ``pattern``: one character per layer for its
    feed-forward (D dense, M mixture of experts, - none); ``v_mix``: one character per layer, 1 = the layer mixes values."""
    layers = []
    for i, fk in enumerate(pattern):
        rot: Dict[str, Any] = {"base": 10000.0, "dims": rot_dims}
        if yarn:
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
        mixer: Dict[str, Any] = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                                 "v_mix": v_mix[i % len(v_mix)] == "1", "mask": {"size": window, "pool": pool}, "rot": rot}
        mlp: Optional[Dict[str, Any]] = None
        if fk == "D":
            mlp = {"kind": "dense", "ff": ff}
        elif fk == "M":
            mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
            if shared_ff:
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Teluzen", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": 1e-5},
            "layers": layers}
