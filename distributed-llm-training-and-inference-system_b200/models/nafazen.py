"""Nafazen: a decoder-only design made of latent-attention mixers (``models/mixers.py``) and dense-xIELU or
mixture-of-experts feed-forwards (``models/ffn.py``) in a post-norm residual layout:

    x <- x + g1 * rmsnorm(mixer(x));   x <- x + g2 * rmsnorm(ff(x))        (g: one number per norm)

The residual stream ``x`` is fp32; sublayers read its rounding to the activation type.  Embeddings are multiplied by
a constant, the final norm has a single gain too, and the logits are soft-capped with tanh.  The layer list, every
size and every constant come from the checkpoint's ``config.json``:

    {"architecture": "Nafazen", "width", "vocab", "embedding": {"scale"}, "norm": {"eps"}, "logit_softcap",
     "layers": [{"type": "latent_attention" | "latent_attention_2",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}?}, "kv_from"?},
                 "mlp": null | {"kind": "dense", "ff"} |
                        {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"}?}}, ...]}

Checkpoint tensors: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,
uv,o}``, ``l<i>.mlp.{up,down,act}`` or ``l<i>.mlp.{router,e<k>.{gate,up,down},shared.{gate,up,down,sg}}``; linear weights
are [out, in].  The model runs ragged paged batches only (``forward_ragged``); the serving engine owns the caches.

Reference: none — the reference serves whatever HF returns (reference llmctl/serve/server.py:127-160)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import elementwise as eops
from ..ops import functional as ops
from .ffn import GatedExpertMoE, XieluMLP
from .mixers import LatentAttention, LatentAttentionSpec
from .registry import Architecture, register_architecture

MIXER_TYPES = ("latent_attention", "latent_attention_2")
YARN_TYPES = ("latent_attention",)      # the second mixer type rotates with the plain frequencies


@dataclass
class NafazenLayer:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[Dict[str, Any]]


@dataclass
class NafazenConfig:
    name: str = "nafazen"
    width: int = 256
    vocab_size: int = 512
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    logit_softcap: Optional[float] = None
    layers: List[NafazenLayer] = field(default_factory=list)
    max_position_embeddings: int = 1 << 20        # rotations are computed from the position; nothing is tabulated
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], name: str = "nafazen") -> "NafazenConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_TYPES:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r} (known: {MIXER_TYPES})")
            m = l["mixer"]
            rot = m["rot"]
            if int(rot["dims"]) != int(m["rot_dim"]) or int(m["rot_dim"]) % 2:
                raise ValueError(f"layer {i}: the rotated part must be rot_dim = rot.dims (even) numbers")
            src = m.get("kv_from")
            spec = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                       kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
                                       rot_base=float(rot["base"]),
                                       rot_scaling=(rot.get("scaling") or None) if l["type"] in YARN_TYPES else None,
                                       kv_from=None if src is None else int(src))
            if src is not None:
                if not 0 <= int(src) < i or layers[int(src)].mixer.kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer that has a cache of its own")
                if layers[int(src)].mixer.cache_width != spec.cache_width:
                    raise ValueError(f"layer {i}: its latent and rope sizes differ from those of layer {src}")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(NafazenLayer(l["type"], spec, mlp))
        cap = d.get("logit_softcap")
        return cls(name=name, width=int(d["width"]), vocab_size=int(d["vocab"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)), logit_softcap=float(cap) if cap else None,
                   layers=layers, raw=d)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def num_parameters(self) -> int:
        n = 0
        with torch.device("meta"):
            m = NafazenModel(self, dtype=torch.bfloat16, device="meta")
        for p in m.parameters():
            n += p.numel()
        return n


class NafazenBlock(nn.Module):
    def __init__(self, cfg: NafazenConfig, layer: NafazenLayer, dtype, device):
        super().__init__()
        W = cfg.width
        self.mixer = LatentAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        self.norm1 = nn.Parameter(torch.ones((), dtype=torch.float32, device=device))
        mlp = layer.mlp
        self.mlp: Optional[nn.Module] = None
        if mlp is not None:
            self.norm2 = nn.Parameter(torch.ones((), dtype=torch.float32, device=device))
            if mlp["kind"] == "dense":
                self.mlp = XieluMLP(W, int(mlp["ff"]), dtype, device)
            else:
                shared = mlp.get("shared")
                self.mlp = GatedExpertMoE(W, int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]),
                                          int(shared["ff"]) if shared else None, dtype, device, scale_input=True,
                                          softmax_scores=False, renormalise=False, shared_gate=True)


class NafazenModel(nn.Module):
    ragged = True           # runs ragged paged batches through ``forward_ragged`` (serve/engine.py)

    def __init__(self, cfg: NafazenConfig, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([NafazenBlock(cfg, l, dtype, device) for l in cfg.layers])
        self.final_norm = nn.Parameter(torch.ones((), dtype=torch.float32, device=device))
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
            self.head.copy_(get("head"))
            self.final_norm.copy_(get("final.norm").float().reshape(()))
            for i, blk in enumerate(self.blocks):
                blk.norm1.copy_(get(f"l{i}.norm1").float().reshape(()))
                blk.mixer.load(get, f"l{i}.mix.")
                if blk.mlp is not None:
                    blk.norm2.copy_(get(f"l{i}.norm2").float().reshape(()))
                    blk.mlp.load(get, f"l{i}.mlp.")

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() == 0:
                    p.fill_(1.0)
                elif p.dim() == 1:
                    p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
                else:
                    fan_in = p.shape[-1]
                    p.copy_((torch.randn(p.shape, generator=g) / fan_in ** 0.5).to(p.dtype))

    # ---- caches ----------------------------------------------------------------------------------------
    def cache_bytes_per_block(self, block_size: int) -> int:
        it = torch.empty((), dtype=self.dtype).element_size()
        return sum(l.mixer.cache_width for l in self.cfg.layers if l.mixer.kv_from is None) * block_size * it

    def allocate_caches(self, num_blocks: int, block_size: int, device) -> List[torch.Tensor]:
        """One ``[blocks, block_size, R + dr]`` tensor per layer that projects its own keys/values; a layer that reads
        another layer's cache gets that very tensor."""
        out: List[Optional[torch.Tensor]] = []
        for l in self.cfg.layers:
            if l.mixer.kv_from is None:
                out.append(torch.zeros(num_blocks, block_size, l.mixer.cache_width, dtype=self.dtype, device=device))
            else:
                out.append(out[l.mixer.kv_from])
        return out

    # ---- forward ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_ragged(self, batch, caches: List[torch.Tensor], layer_trace: Optional[list] = None) -> torch.Tensor:
        """``batch``: serve.ragged.RaggedBatch.  Returns fp32 logits [len(batch.out_rows), vocab]."""
        cfg, dt = self.cfg, self.dtype
        x, h = eops.embed_scale(batch.tokens, self.embed, cfg.embedding_scale)
        for i, blk in enumerate(self.blocks):
            y = blk.mixer(h, batch, caches[i])
            h = eops.postnorm_residual(y, x, blk.norm1, cfg.norm_eps, dt)
            if blk.mlp is not None:
                y = blk.mlp(h, x)
                h = eops.postnorm_residual(y, x, blk.norm2, cfg.norm_eps, dt)
            if layer_trace is not None:
                layer_trace.append(x.clone())
        if batch.num_out == 0:                  # a step that only fills the caches
            return torch.empty(0, cfg.vocab_size, dtype=torch.float32, device=x.device)
        y = eops.scalar_rmsnorm(x, batch.out_rows, self.final_norm, cfg.norm_eps, dt)
        if y.is_cuda and dt == torch.bfloat16 and ops.kernel_config().gemm == "native" and ops._gemm_ok(y, self.head) \
                and self.head.shape[0] % 8 == 0:
            logits = ops.gemm_raw(y, self.head, out_dtype=torch.float32)
        else:
            logits = torch.nn.functional.linear(y, self.head).float()
        if cfg.logit_softcap:
            logits = eops.softcap_(logits.contiguous(), cfg.logit_softcap)
        return logits


def _load_weights(model: NafazenModel, directory) -> None:
    from safetensors.torch import load_file
    model.load_state(load_file(str(Path(directory) / "model.safetensors")))


def build_nafazen(cfg: NafazenConfig, *, dtype=torch.bfloat16, device=None, seed: int = 42, **_ignored) -> NafazenModel:
    m = NafazenModel(cfg, dtype=dtype, device=device)
    m.init_random(seed)
    return m


register_architecture(Architecture(name="Nafazen", config_from_dict=NafazenConfig.from_dict, config_type=NafazenConfig,
                                   build=build_nafazen, load_weights=_load_weights))


def example_config(width: int = 64, vocab: int = 96, heads: int = 2, dim: int = 8, rot_dim: int = 4, vdim: int = 8,
                   kv_rank: int = 16, q_rank: int = 12, ff: int = 48, experts: int = 4, top: int = 2, expert_ff: int = 16,
                   shared_ff: Optional[int] = 24, pattern: str = "aDbMaDcM", yarn: bool = True, softcap: Optional[float] = 20.0,
                   embedding_scale: float = 2.0) -> Dict[str, Any]:
    """A small configuration dictionary for tests, benchmarks and examples.  ``pattern`` is read two characters per
    layer: mixer (a = latent attention with YaRN-scaled rotation, b = plain rotation, c = plain rotation reading the
    cache of the latest b layer) and feed-forward (D dense, M mixture of experts, - none)."""
    layers, last_b = [], None
    for i in range(0, len(pattern), 2):
        mk, fk = pattern[i], pattern[i + 1]
        rot: Dict[str, Any] = {"base": 10000.0 if mk == "a" else 50000.0, "dims": rot_dim}
        if mk == "a" and yarn:
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}
        mixer: Dict[str, Any] = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                                 "rot": rot, "scale": (dim + rot_dim) ** -0.5}
        if mk == "b":
            last_b = len(layers)
        if mk == "c":
            mixer["kv_from"] = last_b
        mlp: Optional[Dict[str, Any]] = None
        if fk == "D":
            mlp = {"kind": "dense", "ff": ff}
        elif fk == "M":
            mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
            if shared_ff:
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "latent_attention" if mk == "a" else "latent_attention_2", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Nafazen", "width": width, "vocab": vocab, "embedding": {"scale": embedding_scale},
            "norm": {"eps": 1e-5}, "logit_softcap": softcap, "layers": layers}
