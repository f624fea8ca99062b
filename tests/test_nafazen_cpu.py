"""Nafazen through the framework (op table, ragged batches, block manager, scheduler, engine) against the plain
oracle in ``nafazen_oracle.py``, on small random configurations.  These run on the CPU implementations of the ops;
``test_nafazen_gpu.py`` repeats the kernel-level and end-to-end comparisons on the CUDA kernels."""
import copy
import json
import math

import pytest
import torch

import nafazen_oracle as oracle

F32 = 2e-4      # fp32 end to end: rounding order only


def make_engine(cfg, weights, dt=torch.float32, device="cpu", blocks=16, bs=8, max_batch=4):
    from llmctl_b200.serve.engine import InferenceEngine
    eng = InferenceEngine(copy.deepcopy(cfg), max_batch_size=max_batch, max_batch_tokens=blocks * bs, device=device,
                          kv_block_size=bs, num_kv_blocks=blocks, dtype=dt, kv_watermark=0.0, cuda_graphs=False)
    eng.model.load_state(weights)
    return eng


def small_cfg(per_layer=None, **kw):
    """``per_layer``: {layer index: mixer keys to override}, so that layers of one model differ in their sizes."""
    from llmctl_b200.models.nafazen import example_config
    cfg = example_config(**kw)
    for i, over in (per_layer or {}).items():
        m = cfg["layers"][i]["mixer"]
        m.update(over)
        if "rot_dim" in over:
            m["rot"]["dims"] = over["rot_dim"]
    return cfg


def run_cut(eng, sid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes; returns logits of every position."""
    out, at = [], 0
    for c in cuts:
        assert eng.kv.allocate(sid, at + c)
        out.append(eng.forward_portions([eng.portion(sid, toks[at:at + c], at, list(range(c)))]))
        at += c
    assert at == len(toks)
    return torch.cat(out)


# ---- mechanisms alone ------------------------------------------------------------------------------------------
def test_rotary_frequencies_and_rotation():
    from llmctl_b200.ops.elementwise import rope_frequencies, rotate_interleaved
    for rot in ({"dims": 8, "base": 10000.0}, {"dims": 16, "base": 5e5, "scaling": {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}},
                {"dims": 2, "base": 100.0, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 2.0}}):
        f, m = rope_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        fo, mo = oracle.rotary_frequencies(rot)
        assert torch.allclose(f, fo, rtol=1e-6, atol=0) and abs(m - mo) < 1e-7
        x = torch.randn(5, 3, rot["dims"])
        pos = torch.tensor([0, 1, 7, 300, 5000])
        assert torch.allclose(rotate_interleaved(x, pos, f, m), oracle.rotate_interleaved(x, pos, rot), atol=1e-5)
    # position 0 is the identity times the amplitude; a pair is turned, not swapped halves
    f, m = rope_frequencies(4, 10.0, None)
    x = torch.tensor([[1.0, 0.0, 0.0, 2.0]])
    r = rotate_interleaved(x, torch.tensor([1]), f, m)
    assert torch.allclose(r[0, :2], torch.tensor([math.cos(1.0), math.sin(1.0)]), atol=1e-6)


def test_scalar_norm_xielu_softcap_embed():
    from llmctl_b200.ops import elementwise as E
    torch.manual_seed(0)
    y, x = torch.randn(6, 10), torch.randn(6, 10)
    g = torch.tensor(0.7)
    want = x + oracle.scalar_norm(y, g, 1e-3)
    E.postnorm_residual(y, x, g, 1e-3, torch.float32)
    assert torch.allclose(x, want, atol=1e-6)
    assert torch.allclose(E.scalar_rmsnorm(x, torch.tensor([4, 1]), g, 1e-3, torch.float32), oracle.scalar_norm(x[[4, 1]], g, 1e-3), atol=1e-6)
    pq = torch.tensor([0.3, -1.2])
    z = torch.linspace(-6, 6, 41)
    assert torch.allclose(E.xielu(z, *E.xielu_coefficients(pq)), oracle.xielu(z, pq), atol=1e-6)
    lg = torch.randn(3, 7) * 50
    assert torch.allclose(E.softcap_(lg.clone(), 20.0), 20.0 * torch.tanh(lg / 20.0), atol=1e-5)
    table = torch.randn(9, 4)
    xs, _ = E.embed_scale(torch.tensor([3, 3, 8]), table, 0.25)
    assert torch.equal(xs, table[[3, 3, 8]] * 0.25)


@pytest.mark.parametrize("top,E,shared", [(1, 4, True), (2, 5, True), (3, 3, False)])
def test_moe_against_oracle(top, E, shared):
    from llmctl_b200.models.ffn import GatedExpertMoE
    torch.manual_seed(1)
    W, ff, sf = 12, 6, 10
    mlp = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff}, "shared": {"ff": sf} if shared else None}
    p = {"router": torch.randn(E, W)}
    for e in range(E):
        p.update({f"e{e}.gate": torch.randn(ff, W) / 3, f"e{e}.up": torch.randn(ff, W) / 3, f"e{e}.down": torch.randn(W, ff) / 3})
    if shared:
        p.update({"shared.gate": torch.randn(sf, W) / 3, "shared.up": torch.randn(sf, W) / 3, "shared.down": torch.randn(W, sf) / 3,
                  "shared.sg": torch.randn(1, W)})
    m = GatedExpertMoE(W, E, top, ff, sf if shared else None, torch.float32, "cpu")
    m.load(lambda k: p[k], "")
    x = torch.randn(9, W)
    assert torch.allclose(m(x, x), oracle.moe_ff(x, p, mlp, True), atol=1e-5)


def test_moe_weight_scales_the_input_not_the_output():
    """With a non-linear expert, expert(w x) != w expert(x): make the router score small so that the two differ much."""
    from llmctl_b200.ops import moe as M
    torch.manual_seed(2)
    W, F = 8, 4
    x = torch.randn(5, W)
    wr = -torch.ones(1, W) * x.sign()[0] * 0.3           # one expert, sigmoid scores well below 1
    wgu, wd = torch.randn(1, 2 * F, W), torch.randn(1, W, F)
    a = M.moe_ffn(x, torch.float32, wr, wgu, wd, 1, scale_input=True)
    b = M.moe_ffn(x, torch.float32, wr, wgu, wd, 1, scale_input=False)
    s = torch.sigmoid(x @ wr.t())
    h = x * s
    want = (torch.nn.functional.silu(h @ wgu[0, :F].t()) * (h @ wgu[0, F:].t())) @ wd[0].t()
    assert torch.allclose(a, want, atol=1e-5) and not torch.allclose(a, b, atol=1e-3)


def test_latent_attention_layer_against_oracle_and_shared_cache():
    """One mixer alone (own cache), and one that reads the first one's cache, fed in two portions."""
    from llmctl_b200.models.mixers import LatentAttention, LatentAttentionSpec
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(3)
    W, T, bs = 20, 13, 4
    mx = {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 10, "q_rank": 7, "scale": 0.4,
          "rot": {"dims": 4, "base": 1000.0, "scaling": {"factor": 4.0, "original": 8, "fast": 4.0, "slow": 1.0}}}
    names = {"dq": (7, W), "dq.norm": (7,), "uq": (3 * 10, 7), "dkv": (14, W), "dkv.norm": (10,), "uk": (18, 10), "uv": (15, 10), "o": (W, 15)}
    p = {k: torch.randn(*s) / 2 for k, s in names.items()}
    p2 = {k: torch.randn(*s) / 2 for k, s in names.items() if not k.startswith("dkv")}
    h = torch.randn(T, W)
    pos = torch.arange(T)
    y_ref, kv = oracle.latent_attention(h, p, mx, pos, 1e-5, True)
    y2_ref, _ = oracle.latent_attention(h, p2, mx, pos, 1e-5, True, shared_kv=kv)
    spec = dict(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=10, q_rank=7, scale=0.4, rot_base=1000.0, rot_scaling=mx["rot"]["scaling"])
    a = LatentAttention(W, LatentAttentionSpec(**spec), 1e-5, torch.float32, "cpu")
    b = LatentAttention(W, LatentAttentionSpec(**spec, kv_from=0), 1e-5, torch.float32, "cpu")
    a.load(lambda k: p[k], "")
    b.load(lambda k: p2[k], "")
    cache = torch.zeros(6, bs, 14)
    table = [5, 2, 0, 3]
    ya, yb = [], []
    for lo, hi in ((0, 6), (6, T)):
        batch = RaggedBatch([Portion(1, [0] * (hi - lo), lo, [], table)], bs, torch.device("cpu"))
        ya.append(a(h[lo:hi], batch, cache))
        yb.append(b(h[lo:hi], batch, cache))
    assert torch.allclose(torch.cat(ya), y_ref, atol=1e-5)
    assert torch.allclose(torch.cat(yb), y2_ref, atol=1e-5)
    # the cache rows are [normed latent | rotated key part] at the table's slots
    rows = cache.view(-1, 14)[torch.tensor([table[j // bs] * bs + j % bs for j in range(T)])]
    assert torch.allclose(rows[:, :10], kv[0], atol=1e-5) and torch.allclose(rows[:, 10:], kv[1], atol=1e-5)


# ---- the model through the engine ---------------------------------------------------------------------------------
CONFIGS = {
    "mixed": dict(),
    # sizes that the usual example makes equal, or 1: one head, top 1, latent wider than the model, no shared expert
    "odd": dict(width=40, heads=1, dim=6, rot_dim=2, vdim=10, kv_rank=48, q_rank=5, ff=20, experts=3, top=1, expert_ff=8,
                shared_ff=None, pattern="bMcDa-", softcap=None, embedding_scale=0.5),
    # every layer with sizes of its own; the layer that reads another's cache shares only its latent and rope sizes
    "per_layer": dict(width=56, heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=24, q_rank=10, pattern="aDbMcDaMc-", top=2, experts=5,
                      per_layer={0: dict(heads=4, rot_dim=8, scale=0.31), 1: dict(heads=2, dim=6, kv_rank=16, rot_dim=6, q_rank=20),
                                 2: dict(heads=5, dim=4, vdim=9, kv_rank=16, rot_dim=6, q_rank=7, scale=0.2),
                                 4: dict(heads=1, dim=10, vdim=3, kv_rank=16, rot_dim=6, q_rank=33)}),
    "many_heads": dict(width=48, heads=5, dim=4, rot_dim=6, vdim=3, kv_rank=9, q_rank=16, experts=6, top=3, pattern="aMbDcMcD", yarn=False),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_layer_trace(name):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, seed=11)
    toks = torch.randint(0, cfg["vocab"], (45,), generator=torch.Generator().manual_seed(1)).tolist()
    tr = []
    ref = oracle.forward(cfg, w, toks, exact=True, trace=tr)
    eng = make_engine(cfg, w)
    assert eng.kv.allocate(1, len(toks))
    mine = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=mine)
    for i, (a, b) in enumerate(zip(mine, tr)):
        assert torch.allclose(a, b, atol=F32), f"residual stream differs after layer {i}"
    assert torch.allclose(got, ref, atol=F32)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_portions_and_decode_agree(name):
    """Token-by-token decoding, portions down to two tokens cut inside pages, and one whole prompt give the oracle's
    logits at every position (block size 8, prompt over several pages)."""
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, seed=12)
    toks = torch.randint(0, cfg["vocab"], (61,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = oracle.forward(cfg, w, toks, exact=True)
    eng = make_engine(cfg, w)
    for sid, cuts in enumerate(([1] * 61, [2, 5, 8, 1, 17, 2, 2, 16, 3, 1, 1, 1, 1, 1], [7, 54], [60, 1]), start=1):
        got = run_cut(eng, sid, toks, cuts)
        assert torch.allclose(got, ref, atol=F32), f"cuts {cuts[:4]}..."
        eng.kv.free(sid)


def test_unequal_batch_matches_each_alone_and_pages_are_reused():
    """Four live requests of unequal length advance in mixed batches (portions next to single tokens, some skipping a
    step) in a pool that only holds them because finished requests give their pages back."""
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=13)
    g = torch.Generator().manual_seed(3)
    lens = [50, 9, 33, 1, 26, 40, 17]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    refs = [oracle.forward(cfg, w, r, exact=True) for r in reqs]
    eng = make_engine(cfg, w, blocks=18, bs=8)          # 144 token slots < sum(lens) = 176
    waiting, live, done, step = list(range(len(reqs))), {}, 0, 0
    owners_of_block = {}
    while waiting or live:
        while waiting and len(live) < 4 and eng.kv.free_blocks * 8 >= lens[waiting[0]] + 8:
            live[waiting.pop(0)] = 0
        portions, owners = [], []
        for k, (i, at) in enumerate(sorted(live.items())):
            if (step + i) % 5 == 4:
                continue                                  # left out of this step
            n = min([1, 2, 11, 1, 5][(step + k) % 5], lens[i] - at) if at else min(3 + 4 * k, lens[i])
            assert eng.kv.allocate(100 + i, at + n)
            for blk in eng.kv.block_table(100 + i):
                owners_of_block.setdefault(blk, set()).add(i)
            portions.append(eng.portion(100 + i, reqs[i][at:at + n], at, list(range(n))))
            owners.append((i, at, n))
        if portions:
            lg = eng.forward_portions(portions)
            o = 0
            for i, at, n in owners:
                assert torch.allclose(lg[o:o + n], refs[i][at:at + n], atol=F32), f"request {i} at {at} (+{n}) in step {step}"
                o += n
                live[i] = at + n
                if at + n == lens[i]:
                    eng.kv.free(100 + i)
                    del live[i]
                    done += 1
        step += 1
        assert step < 400
    assert done == len(reqs) and eng.kv.free_blocks == 18
    assert sum(len(v) > 1 for v in owners_of_block.values()) >= 4, "pages were not handed out again"


def test_far_key_is_found_across_pages():
    """One key far back decides the output: scale the matching query and key so that its score stands out, and check
    that decoding through the cache finds it at a page border, mid-page and at position 0."""
    from llmctl_b200.ops import latent_attention as L
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(4)
    H, R, dr, dn, bs, n = 2, 6, 2, 3, 8, 300
    f = torch.tensor([1.0])
    cache = torch.zeros(40, bs, R + dr)
    table = torch.randperm(40).tolist()[:38]
    rows = torch.randn(n, R + dr) * 0.1
    for far in (0, 7, 8, 130, 255, 256):
        r = rows.clone()
        r[far, :R] = torch.tensor([9.0, 0, 0, 0, 0, 0])
        r[far, R:] = 0
        slots = torch.tensor([table[j // bs] * bs + j % bs for j in range(n)])
        cache.view(-1, R + dr)[slots] = r
        ql = torch.zeros(1, H, R)
        ql[0, :, 0] = 9.0
        q = torch.zeros(1, H * (dn + dr))
        b = RaggedBatch([Portion(1, [0], n - 1, [], table)], bs, torch.device("cpu"))
        out = L.latent_attention(ql, q, dn, cache, b.block_tables, b.tiles(), b.positions, f, 1.0, 1.0, b.heads_per_tile(H), n)
        assert torch.allclose(out[0, 0], r[far, :R], atol=1e-3), f"far key at {far}"


def test_long_decode_through_engine_scheduler_is_greedy_consistent():
    """Greedy generation through ``InferenceEngine.generate`` (scheduler, block growth, batched decode of unequal
    requests): every generated token is the argmax of the oracle run on the tokens before it."""
    cfg = small_cfg(pattern="aDbMcM", softcap=None)
    w = oracle.random_weights(cfg, seed=14)
    eng = make_engine(cfg, w, blocks=40, bs=8)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 19, 1)]
    outs = eng.generate(prompts, max_tokens=40, temperature=0.0)
    for p, o in zip(prompts, outs):
        assert len(o) == 40
        ref = oracle.forward(cfg, w, p + o, exact=True)
        top2 = ref.topk(2, -1).values
        for k, tok in enumerate(o):
            row = len(p) + k - 1
            if top2[row, 0] - top2[row, 1] > 1e-3:          # skip near ties
                assert tok == int(ref[row].argmax()), f"token {k} of prompt len {len(p)}"
    assert eng.kv.free_blocks == 40


def test_config_reader_and_registry(tmp_path):
    from safetensors.torch import save_file
    from llmctl_b200.models.config import resolve_model
    from llmctl_b200.models.nafazen import NafazenConfig
    from llmctl_b200.serve.engine import InferenceEngine
    cfg = small_cfg(pattern="bDcM")
    w = oracle.random_weights(cfg, seed=15)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    c = resolve_model(tmp_path)
    assert isinstance(c, NafazenConfig) and c.layers[1].mixer.kv_from == 0 and c.layers[0].mlp["kind"] == "dense"
    eng = InferenceEngine(tmp_path, device="cpu", kv_block_size=8, num_kv_blocks=8, dtype=torch.float32)
    toks = [1, 2, 3, 4, 5]
    assert eng.kv.allocate(1, 5)
    got = eng.forward_portions([eng.portion(1, toks, 0, [4])])
    assert torch.allclose(got[0], oracle.forward(cfg, w, toks)[4], atol=F32)
    bad = copy.deepcopy(cfg)
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ValueError):
        NafazenConfig.from_dict(bad)
    bad = copy.deepcopy(cfg)
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        NafazenConfig.from_dict(bad)


def test_trace_replay_steps(tmp_path):
    """The replayer admits requests at their first entry, lets one skip a step, frees pages at ``end`` and writes
    logits in entry order."""
    from safetensors.torch import save_file
    from llmctl_b200.serve.replay import TraceReplayer
    cfg = small_cfg(pattern="aDbM")
    w = oracle.random_weights(cfg, seed=16)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    a = list(range(3, 80))
    b = list(range(40, 50))
    ra, rb = oracle.forward(cfg, w, a), oracle.forward(cfg, w, b)
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens=192, device="cpu")      # three pages of 64: a holds two, b one
    l0 = rp.step({"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []})
    assert torch.allclose(l0, torch.stack([ra[0], ra[69], rb[1]]), atol=F32)
    assert rp.step({"step": 1, "entries": [{"id": "b", "tokens": b[2:9], "want": []}], "end": []}) is None
    l2 = rp.step({"step": 2, "entries": [{"id": "b", "tokens": b[9:], "want": [0]}, {"id": "a", "tokens": a[70:], "want": [6]}], "end": ["a", "b"]})
    assert torch.allclose(l2, torch.stack([rb[9], ra[76]]), atol=F32)
    assert rp.engine.kv.free_blocks == 3 and not rp.live
    # the freed pages serve a new request
    l3 = rp.step({"step": 3, "entries": [{"id": "c", "tokens": a, "want": [76]}, {"id": "d", "tokens": b, "want": [9]}], "end": ["c"]})
    assert torch.allclose(l3, torch.stack([ra[76], rb[9]]), atol=F32)
    with pytest.raises(RuntimeError):           # d still holds a page: two more requests of two pages do not fit
        rp.step({"step": 4, "entries": [{"id": "e", "tokens": a, "want": []}, {"id": "f", "tokens": a, "want": []}], "end": []})


def test_bfloat16_serving_precision_is_close_to_oracle():
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=17)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(6)).tolist()
    ref = oracle.forward(cfg, w, toks, exact=True)
    eng = make_engine(cfg, w, dt=torch.bfloat16)
    got = run_cut(eng, 1, toks, [25] + [1] * 15)
    err = (got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()
    assert err < 0.05, err
