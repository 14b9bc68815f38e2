"""The Gerupel design in the engine against the plain numpy statement of it (tests/plain/gerupel_plain.py).

Every test makes its own small configuration and random weights.  Each body runs twice: with the PyTorch stand-ins
for the kernels on the CPU (the parts, the cache manager, the batching), and on the GPU with the real kernels (marked
``gpu``).  The configurations differ from one another in everything a configuration can say: which layers run again and
how often, windows shorter and longer than the pooled blocks, a window and blocks of one token, a layer without a mask,
without a rotation, without a frequency scaling or without a feed-forward, grouped and ungrouped heads, key, value and
rotated sizes that differ, routers that choose one, some or all of their experts.
"""

import json
import os

import numpy as np
import pytest
import torch

import sllm_b200.models  # noqa: F401  (registers the parts and the architecture)
from tests import traces
from tests.plain import gerupel_plain as plain


def _left(heads, kv, dim, vdim, scale, size=None, pool=None, rot=None, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size, "pool": pool}
    if rot is not None:
        m["rot"] = {"base": base, "dims": rot, "scaling": scaling}
    return m


def _mixer(left, right, ls, rs):
    return {"left": left, "right": dict(zip(("heads", "dim", "vdim"), right)), "left_scale": ls, "right_scale": rs}


def _moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


SCALING = {"factor": 3.0, "low": 1.0, "high": 6.0, "original": 64}

CONFIG_A = {          # the middle layers run twice; a window shorter than its blocks; a layer without a feed-forward
    "architecture": "Gerupel", "vocab": 300, "width": 96, "residual_mult": 0.4, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "parallel", "mixer": _mixer(_left(4, 2, 24, 16, 0.2, 12, 5, rot=8, scaling=SCALING), (3, 8, 20), 1.3, 0.6), "mlp": _moe(5, 2, 40, 1.5)},
        {"type": "parallel", "mixer": _mixer(_left(2, 1, 16, 32, 0.25, 6, 9, rot=16, base=500.0), (2, 16, 16), 0.7, 1.1), "mlp": None},
        {"type": "parallel", "mixer": _mixer(_left(6, 3, 16, 16, 0.3, 20, 4, rot=12, scaling=SCALING), (1, 24, 40), 1.0, 1.0), "mlp": _moe(4, 1, 24, 0.8)},
        {"type": "parallel", "mixer": _mixer(_left(3, 3, 32, 24, 0.15, 9, 2), (4, 6, 10), 0.9, 0.4), "mlp": _moe(6, 3, 16, 2.0)},
    ],
}
CONFIG_B = {          # heads of 64 on pages of 16 (the tensor-core attention forms on the GPU in bfloat16); the first layer runs three times
    "architecture": "Gerupel", "vocab": 200, "width": 128, "residual_mult": 0.5, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 1, "times": 3},
    "layers": [
        {"type": "parallel", "mixer": _mixer(_left(8, 2, 64, 64, 0.11, 32, 8, rot=16, scaling={"factor": 8.0, "low": 1.0, "high": 6.0, "original": 96}),
                                             (2, 32, 48), 1.1, 0.7), "mlp": _moe(8, 2, 32, 1.8)},
        {"type": "parallel", "mixer": _mixer(_left(4, 4, 64, 32, 0.11, 24, 16, rot=64), (4, 16, 16), 1.0, 0.8), "mlp": _moe(4, 4, 64, 1.0)},
        {"type": "parallel", "mixer": _mixer(_left(6, 1, 32, 64, 0.18, 48, 12, rot=8, base=100.0), (1, 64, 64), 0.6, 1.4), "mlp": None},
    ],
}
ODD = {               # sizes that are multiples of nothing; a window and blocks of ONE token (every older token is a block); no mask at all
    "architecture": "Gerupel", "vocab": 77, "width": 50, "residual_mult": 1.0, "norm": {"eps": 1e-4},
    "layers": [
        {"type": "parallel", "mixer": _mixer(_left(3, 1, 10, 14, 0.4, 1, 1, rot=6, base=50.0), (5, 6, 7), 1.0, 1.0), "mlp": _moe(3, 3, 14, 0.7)},
        {"type": "parallel", "mixer": _mixer(_left(1, 1, 12, 9, 0.3, rot=4, base=50.0), (1, 20, 7), 2.0, 0.3), "mlp": _moe(1, 1, 18, 1.1)},
        {"type": "parallel", "mixer": _mixer(_left(5, 5, 6, 6, 0.5, 7, 3), (2, 9, 11), 0.5, 0.5), "mlp": _moe(7, 1, 9, 1.0)},
    ],
}
LOOP_ALL = {          # every layer in the loop, five passes; blocks as long as the window
    "architecture": "Gerupel", "vocab": 120, "width": 64, "residual_mult": 0.2, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 5},
    "layers": [
        {"type": "parallel", "mixer": _mixer(_left(2, 2, 16, 16, 0.25, 8, 8, rot=16), (2, 8, 8), 1.0, 1.0), "mlp": _moe(16, 5, 8, 1.0)},
        {"type": "parallel", "mixer": _mixer(_left(4, 1, 32, 16, 0.2, 16, 3, rot=8, scaling=SCALING), (1, 32, 32), 1.5, 0.5), "mlp": _moe(2, 1, 48, 3.0)},
    ],
}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 16), "odd": (ODD, 8), "loop_all": (LOOP_ALL, 4)}


def _devices():
    return [pytest.param("cpu", id="stand-in"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]


@pytest.fixture(params=_devices())
def dev(request):
    if request.param == "cpu":
        request.getfixturevalue("cpu_ops")
    elif not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return request.param


def make_model(tmp_path, config, seed=5, name="m", edit=None, std=0.12):
    from sllm_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    d = write_random_model(os.path.join(str(tmp_path), name), config, seed, std=std, bias_std=0.4, gain_std=0.2)
    if edit is not None:
        f = SafetensorsFile(os.path.join(d, "model.safetensors"))
        t = {n: f.tensor(n).float() for n in f.names()}
        edit(t)
        del f
        write_safetensors(os.path.join(d, "model.safetensors"), {n: v.to(torch.bfloat16) for n, v in t.items()})
    return d


def plain_logits(d, reqs, margins=None):
    cfg, w = plain.load_model(d)
    out = {}
    for r, ids in reqs.items():
        m = []
        out[r] = plain.forward(cfg, w, ids, margins=m).astype(np.float32)
        if margins is not None:
            margins[r] = np.min(np.stack(m), axis=0) if m else np.full(len(ids), np.inf)
    return out


def dtypes_on(dev):
    return ("float32",) if dev == "cpu" else ("float32", "bfloat16")


def models_for(tmp_path, config, dev, reqs, seed=5, edit=None):
    for dtype in dtypes_on(dev):
        d = make_model(tmp_path, config, seed=seed, name=f"m_{dtype}", edit=edit)
        margins = {}
        yield dtype, d, plain_logits(d, reqs, margins), margins


CLOSE_CALL = 0.04


def compare(tr, out, want, dtype, what, margins=None, sharp=False):
    """float32: every logit to 3e-4.  bfloat16: the difference of a row (mean taken off, root mean square over the
    vocabulary) relative to the row's own spread is rounding's: under 4 % for 19 rows in 20 and under 15 % for every
    row; rows whose routers decided on a close call (``margins`` under `CLOSE_CALL`) are left out there, since bfloat16
    rounding may send such a token to another expert, which is no fault.  ``sharp``: the weights were sharpened so that one
    lost key or block changes a row by its whole spread; rounding grows with them, and the bounds are twice as wide."""
    if dtype == "float32":
        return traces.compare(tr, out, want, what=what, rtol=3e-4, atol=3e-4)
    most, every = (0.08, 0.3) if sharp else (0.04, 0.15)
    errs, skipped = [], 0
    for s in tr.steps:
        for row, (req, pos) in enumerate(s["expect"]):
            if margins is not None and margins[req.split(".")[-1]][pos] < CLOSE_CALL:
                skipped += 1
                continue
            ref, got = want[req][pos], out[s["step"]][row]
            d, r = got - ref, ref - ref.mean()
            e = float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((r ** 2).mean()))
            assert e < every, f"{what}: step {s['step']}, request {req!r}, position {pos}: relative difference {e:.3g}"
            errs.append(e)
    # (a model whose layers run five times asks ten routers per token: most rows then hold some close call; twenty rows are still a comparison)
    assert skipped <= len(errs) or len(errs) >= 20, f"{what}: {skipped} rows left out for close calls, {len(errs)} compared"
    assert np.quantile(errs, 0.95) < most, f"{what}: 95th percentile of the rows' relative difference {np.quantile(errs, 0.95):.3g}"


def _requests(vocab, lengths, seed=3):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(lengths)}


def _to(dev):
    return lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).contiguous()


def _bf16_exact(w):
    return {n: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64) for n, a in w.items()}


def _i32(dev, v):
    return torch.tensor(np.asarray(v).tolist(), dtype=torch.int32, device=dev)


def _step(dev, q_lens, slots, ctx_lens=None, groups=()):
    """A batch description by hand: portions of ``q_lens`` tokens that end at ``ctx_lens`` (default: start at 0)."""
    from sllm_b200.parts import StepContext
    ctx_lens = list(ctx_lens or q_lens)
    starts = np.concatenate([[0], np.cumsum(q_lens)])
    pos = np.concatenate([np.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)])
    return StepContext(num_tokens=int(starts[-1]), num_seqs=len(q_lens), token_ids=_i32(dev, [0] * int(starts[-1])), positions=_i32(dev, pos),
                       seq_of_token=_i32(dev, np.repeat(np.arange(len(q_lens)), q_lens)), q_start=_i32(dev, starts),
                       ctx_len=_i32(dev, ctx_lens), state_slots=_i32(dev, slots), logit_rows=_i32(dev, []), groups=list(groups),
                       q_lens=list(q_lens), ctx_lens=ctx_lens, max_q_len=max(q_lens), max_ctx_len=max(ctx_lens))


# ---- configuration, plan, cache needs ---------------------------------------------------------------------------

def test_config_plan_and_cache_needs():
    from sllm_b200.config import ConfigError, architecture_of
    from sllm_b200.models.causal_lm import CausalLM
    from sllm_b200.parts import PagedKV, SlotState
    arch = architecture_of(CONFIG_A)
    cfg = arch.config_cls.from_dict(CONFIG_A)
    assert cfg.to_dict() == CONFIG_A
    p = arch.plan(cfg)
    assert [(e.layer, e.reentry) for e in p.run_list] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert p.head_name is None and p.embedding_norm is not None and p.pass_vectors_name == "loop.step" and p.passes == 2
    assert [(e.layer, e.reentry) for e in arch.plan(arch.config_cls.from_dict(ODD)).run_list] == [(0, None), (1, None), (2, None)]
    assert [(e.layer, e.reentry) for e in arch.plan(arch.config_cls.from_dict(CONFIG_B)).run_list] == [(0, 0), (0, 1), (0, 2), (1, None), (2, None)]
    m = CausalLM(p, dtype=torch.float32, device="cpu")
    needs = m.cache_needs()
    assert len(needs) == 6
    # tokens are kept for as long as the window or a block's means need them; the blocks' means for good, one per block
    assert needs[0] == ("own", (PagedKV(2, 24, 12), PagedKV(2, 24, None, stride=5, name="pooled"), SlotState((3, 8, 20), "forget_gate")))
    assert needs[1] == needs[3] == ("own", (PagedKV(1, 32, 9), PagedKV(1, 32, None, stride=9, name="pooled"), SlotState((2, 16, 16), "forget_gate")))
    odd = CausalLM(arch.plan(arch.config_cls.from_dict(ODD)), dtype=torch.float32, device="cpu").cache_needs()
    assert odd[1] == ("own", (PagedKV(1, 12, None), SlotState((1, 20, 7), "forget_gate")))          # no mask: all keys, no blocks
    shapes = {s.name: tuple(s.shape) for s in m.tensor_specs()}
    assert shapes["embed.norm"] == (96,) and shapes["loop.step"] == (2, 96) and shapes["l0.mix.left.temp"] == (4,)
    assert shapes["l0.mix.left.q"] == (96, 96) and shapes["l0.mix.left.k"] == (48, 96) and shapes["l0.mix.left.v"] == (32, 96)
    assert shapes["l0.mix.left.o"] == (96, 64) and shapes["l0.mix.right.q"] == (24, 96) and shapes["l0.mix.right.f.b"] == (24,)
    assert shapes["l0.mix.right.lower"] == (24,) and shapes["l0.mix.right.norm"] == (20,) and shapes["l0.mix.right.o"] == (96, 60)
    assert shapes["l0.mlp.router"] == (5, 96) and shapes["l0.mlp.e4.down"] == (96, 40) and "head" not in shapes
    assert not any(n.startswith(("l1.mlp", "l1.norm2")) for n in shapes)

    def edited(path, value):
        c = json.loads(json.dumps(CONFIG_A))
        at = c
        for k in path[:-1]:
            at = at[k]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        return c
    for bad in (edited(("layers", 0, "mlp", "router", "top"), 6), edited(("layers", 0, "type"), "other"),
                edited(("layers", 0, "mlp", "kind"), "dense"), edited(("layers", 0, "mixer", "left", "kv_heads"), 3),
                edited(("layers", 0, "mixer", "left", "rot", "dims"), 26), edited(("layers", 0, "mixer", "left", "rot", "dims"), 7),
                edited(("loop", "stop"), 5), edited(("loop", "start"), 4), edited(("loop", "times"), 0),
                edited(("layers", 0, "mixer", "right_scale"), None), edited(("norm",), None)):
        with pytest.raises(ConfigError):
            arch.config_cls.from_dict(bad)


def test_pages_of_one_entry_per_block_in_the_cache_manager_and_the_packer():
    """A cache group that holds one entry per block of tokens: how many pages a request needs, where the token that
    completes a block writes, what goes back when, and that the tokens' pages behind the window AND the block are let go."""
    from sllm_b200.cache.manager import CacheManager
    from sllm_b200.engine.batch import BatchLayout, pack
    from sllm_b200.engine import StepEntry
    from sllm_b200.parts import PagedKV
    needs = [("own", (PagedKV(1, 8, 6), PagedKV(1, 8, None, stride=5, name="pooled")))]
    cm = CacheManager(needs, page_size=4, num_pages=[8, 3], max_requests=2)
    assert [cm.pages_for(n, 1) for n in (0, 4, 5, 19, 20, 24, 25, 45)] == [0, 0, 1, 1, 1, 1, 2, 3] and cm.tokens_per_page(1) == 20
    assert cm.fits_at_all(60) and not cm.fits_at_all(80)                  # 16 entries need four pages of the pooled group's three
    with pytest.raises(TypeError):
        CacheManager([("own", PagedKV(1, 8, 6, stride=5))], page_size=4, num_pages=4, max_requests=1)      # a window on pooled entries
    with pytest.raises(TypeError):
        CacheManager([("own", (PagedKV(1, 8, 6), PagedKV(1, 8, None)))], page_size=4, num_pages=4, max_requests=1)   # two of one name
    cm.add_request("a")
    cm.reserve("a", 13)
    req = cm.requests["a"]
    assert len(req.tables[0]) == 4 and len(req.tables[1]) == 1
    e = StepEntry("a", list(range(13)), [12])
    lay = BatchLayout(13, 1, 1, [4, 1])
    h = np.zeros(lay.total, dtype=np.int32)
    pack(lay, h, cm, [e], [13])
    pooled = lay.sec(h, "slot_mapping1")
    page = req.tables[1][0]
    assert pooled.tolist() == [-1, -1, -1, -1, page * 4, -1, -1, -1, -1, page * 4 + 1, -1, -1, -1]
    cm.commit("a", 13)
    assert req.tables[0][:2] == [-1, -1] and req.tables[0][2] >= 0 and req.tables[1][0] == page      # positions 0..7 lie behind window and block
    cm.reserve("a", 27)
    e = StepEntry("a", list(range(14)), [])
    lay = BatchLayout(14, 1, 0, [7, 2])
    h = np.zeros(lay.total, dtype=np.int32)
    pack(lay, h, cm, [e], [27])
    p2 = req.tables[1][1]
    assert [int(s) for s in lay.sec(h, "slot_mapping1") if s >= 0] == [page * 4 + 2, page * 4 + 3, p2 * 4]     # blocks 2, 3 and 4
    assert lay.sec(h, "block_tables1").tolist() == [page, p2]
    cm.commit("a", 27)
    cm.check()
    assert cm.token_room("a") == min((7 + cm.groups[0].pool.free_count) * 4, (2 + 1) * 20)
    cm.free_request("a")
    cm.check()
    assert all(g.pool.used_count == 0 for g in cm.groups)


# ---- each mechanism alone ------------------------------------------------------------------------------------------

def test_rotation_frequencies_in_three_regimes():
    from sllm_b200.parts.standard import Rotary
    for base, dims, sc in ((10000.0, 24, {"factor": 6.0, "low": 1.0, "high": 8.0, "original": 256}), (500.0, 8, SCALING), (100.0, 64, None),
                           (10000.0, 16, {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 40})):
        f, mag = Rotary.frequencies(base, dims, sc)
        want = plain.rotary_frequencies(base, dims, sc)
        np.testing.assert_allclose(f, want, rtol=1e-13)
        assert mag == 1.0
        if sc:                                                # all three regimes occur, or the case tests nothing
            wave = 2 * np.pi / plain.rotary_frequencies(base, dims)
            assert (wave < sc["original"] / sc["high"]).any() and (wave > sc["original"] / sc["low"]).any()
    wave = 2 * np.pi / plain.rotary_frequencies(500.0, 8)
    assert ((wave >= SCALING["original"] / SCALING["high"]) & (wave <= SCALING["original"] / SCALING["low"])).any()


@pytest.mark.parametrize("W", (50, 96, 2304))
def test_two_norms_of_one_row_and_what_a_pass_takes_in(dev, W):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(W)
    x = rng.standard_normal((7, W)) * 3.0
    ga, gb = rng.standard_normal(W), rng.standard_normal(W)
    a, b = ops.norm_pair(_to(dev)(x), _to(dev)(ga), _to(dev)(gb), 1e-5, torch.float32)
    np.testing.assert_allclose(a.cpu().numpy(), plain.rms_norm(x, ga, 1e-5), rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(b.cpu().numpy(), plain.rms_norm(x, gb, 1e-5), rtol=2e-6, atol=2e-6)
    a, b = ops.norm_pair(_to(dev)(x), _to(dev)(ga), None, 1e-5, torch.float32)
    assert b is None
    np.testing.assert_allclose(a.cpu().numpy(), plain.rms_norm(x, ga, 1e-5), rtol=2e-6, atol=2e-6)
    s, rows, vec = _to(dev)(x), rng.standard_normal((7, W)), rng.standard_normal(W)
    ops.add_rows_(s, _to(dev)(rows), _to(dev)(vec))
    np.testing.assert_allclose(s.cpu().numpy(), x + rows + vec, rtol=2e-6, atol=2e-6)
    ops.add_rows_(s, None, _to(dev)(vec))
    np.testing.assert_allclose(s.cpu().numpy(), x + rows + 2 * vec, rtol=2e-6, atol=2e-6)


def _paged(dev, seqs, G, D, ps, stride, dtype, rng):
    """Pages for sequences of ``seqs`` tokens (one entry per ``stride`` of them) under shuffled page ids: (k pages, v pages,
    block tables as a list of lists)."""
    counts = [-(-(n // stride) // ps) for n in seqs]
    ids = rng.permutation(sum(counts) + 3).tolist()
    tables, at = [], 0
    for c in counts:
        tables.append(ids[at:at + c])
        at += c
    shape = (sum(counts) + 3, G, ps, D)
    return torch.full(shape, float("nan"), dtype=dtype, device=dev), torch.full(shape, float("nan"), dtype=dtype, device=dev), tables


def _pooled_case(dev, seqs, H, G, D, vdim, window, pool, ps, dtype, cuts, seed=0, standout=None):
    """Keys and values of several sequences written into shuffled pages portion by portion (``cuts``: tokens of each
    sequence per step); every step pools what it completes and attends; returns (got, want) per sequence, [n, H, vdim]."""
    import sllm_b200.ops as ops
    from sllm_b200.parts.base import GroupView
    rng = np.random.default_rng(seed)
    q = [rng.standard_normal((n, H, D)) for n in seqs]
    k = [rng.standard_normal((n, G, D)) for n in seqs]
    v = [rng.standard_normal((n, G, D)) for n in seqs]
    for vv in v:
        vv[..., vdim:] = 0.0
    if standout is not None:
        standout(q, k, v)
    cast = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype)
    exact = lambda a: cast(a).float().numpy().astype(np.float64)
    q, k, v = [exact(a) for a in q], [exact(a) for a in k], [exact(a) for a in v]
    kc, vc, tk = _paged(dev, seqs, G, D, ps, 1, dtype, rng)
    pk, pv, tp = _paged(dev, seqs, G, D, ps, pool, dtype, rng)
    width = lambda t: max(max(len(r) for r in t), 1)
    table = lambda t, live: _i32(dev, [t[s] + [-1] * (width(t) - len(t[s])) for s in live])
    scale = 0.3
    at, got = [0] * len(seqs), [[] for _ in seqs]
    for cut in cuts:
        live = [s for s in range(len(seqs)) if at[s] < seqs[s]]
        if not live:
            break
        n = [min(cut[s % len(cut)], seqs[s] - at[s]) for s in live]
        pos = [np.arange(at[s], at[s] + m) for s, m in zip(live, n)]
        slot_k = np.concatenate([[tk[s][p // ps] * ps + p % ps for p in pp] for s, pp in zip(live, pos)])
        slot_p = np.concatenate([[tp[s][(p + 1) // pool // ps - (0 if ((p + 1) // pool) % ps else 1)] * ps + ((p + 1) // pool - 1) % ps
                                  if (p + 1) % pool == 0 else -1 for p in pp] for s, pp in zip(live, pos)])
        for s, pp in zip(live, pos):                        # the tokens' keys and values go to their pages (what the rotary kernel does)
            for p in pp:
                kc[tk[s][p // ps], :, p % ps, :] = cast(k[s][p]).to(dev)
                vc[tk[s][p // ps], :, p % ps, :] = cast(v[s][p]).to(dev)
        groups = [GroupView(ps, table(tk, live), _i32(dev, slot_k)), GroupView(ps, table(tp, live), _i32(dev, slot_p))]
        step = _step(dev, n, list(range(len(live))), [at[s] + m for s, m in zip(live, n)], groups)
        ops.pool_kv_write(kc, vc, step, 0, pk, pv, 1, pool)
        qq = cast(np.concatenate([q[s][pp] for s, pp in zip(live, pos)]).reshape(-1, H * D)).to(dev).contiguous()
        sink = torch.zeros(H, dtype=torch.float32, device=dev)
        o = ops.pooled_attention(qq, kc, vc, pk, pv, step, 0, 1, H, G, vdim, scale, window, pool, sink, 1.0).float().cpu().numpy()
        r0 = 0
        for s, m in zip(live, n):
            got[s].append(o[r0:r0 + m].reshape(m, H, vdim))
            r0 += m
            at[s] += m
    want = []
    for s in range(len(seqs)):
        kk = k[s] if dtype == torch.float32 else None
        if kk is None:                                      # bfloat16: the blocks' means are rounded as the pages hold them
            want.append(_plain_pooled_rounded(q[s], k[s], v[s], scale, window, pool, vdim))
        else:
            want.append(plain.pooled_window_attention(q[s], k[s], v[s][..., :vdim], scale, np.ones(H), window, pool))
    return [np.concatenate(g) for g in got], want


def _plain_pooled_rounded(q, k, v, scale, window, pool, vdim):
    """The plain attention with each block's means rounded to bfloat16, as a bfloat16 cache holds them: block b stands in
    for its tokens as ONE token whose key and value are those means."""
    T, H, D = q.shape
    G = k.shape[1]
    rnd = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)
    nb = T // pool
    pk = rnd(np.stack([k[b * pool:(b + 1) * pool].mean(0) for b in range(nb)])) if nb else np.zeros((0, G, D))
    pv = rnd(np.stack([v[b * pool:(b + 1) * pool].mean(0) for b in range(nb)])) if nb else np.zeros((0, G, D))
    out = np.zeros((T, H, vdim))
    for i in range(T):
        lo = max(0, i - window + 1)
        n = lo // pool
        for h in range(H):
            g = h // (H // G)
            keys, vals = np.concatenate([pk[:n, g], k[lo:i + 1, g]]), np.concatenate([pv[:n, g], v[lo:i + 1, g]])
            s = keys @ q[i, h] * scale
            m = max(float(s.max()), 0.0)
            e = np.exp(s - m)
            out[i, h] = (e[:, None] * vals[:, :vdim]).sum(0) / (np.exp(-m) + e.sum())
    return out


ATT_CUTS = [(40, 1, 7), (1, 2, 30), (2, 9, 1), (13, 1, 1), (1, 1, 64), (300, 300, 300)]


@pytest.mark.parametrize("H,G,D,vdim,window,pool,ps", [(4, 2, 16, 16, 12, 5, 8), (3, 3, 24, 10, 6, 9, 4), (8, 1, 64, 64, 32, 8, 16),
                                                       (2, 1, 40, 40, 1, 1, 16), (6, 2, 128, 96, 44, 12, 16), (2, 2, 200, 7, 16, 16, 32)])
def test_window_and_pooled_blocks_in_portions_and_single_tokens(dev, H, G, D, vdim, window, pool, ps):
    """Portions of many sizes beside single tokens, three sequences in shuffled pages (pages nobody wrote hold NaN): every
    query's window edge, every block's first appearance, and the sequence's first tokens are among the rows compared."""
    for dtype in ((torch.float32,) if dev == "cpu" or D > 128 else (torch.float32, torch.bfloat16)):
        got, want = _pooled_case(dev, (150, 97, 33), H, G, D, vdim, window, pool, ps, dtype, ATT_CUTS, seed=D + pool)
        tol = 3e-5 if dtype == torch.float32 else 2e-2
        for g, w in zip(got, want):
            assert np.isfinite(g).all()
            np.testing.assert_allclose(g, w, rtol=tol, atol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("D,vdim,window,pool", [(64, 64, 200, 4), (128, 96, 330, 3), (32, 32, 70, 1)])
def test_single_tokens_over_many_tiles_cut_into_runs(D, vdim, window, pool):
    """Decoded tokens far into a sequence: the 16-row tensor-core form cuts the tiles of blocks' entries and of the window's
    tokens into runs for CTAs of their own and merges them; two requests of unequal length side by side."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sllm_b200.ops as ops
    assert ops.pooled_splits(2, 2, 900, window, pool) > 1
    cuts = [(880, 500)] + [(1, 1)] * 8 + [(12, 1)]
    got, want = _pooled_case("cuda:0", (900, 509), 4, 2, D, vdim, window, pool, 16, torch.bfloat16, cuts, seed=D)
    for g, w in zip(got, want):
        np.testing.assert_allclose(g[-20:], w[-20:], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("window,pool,ps", [(12, 5, 8), (36, 12, 16), (8, 8, 4), (5, 13, 16)])
def test_a_key_that_stands_out_just_inside_and_outside_the_window_and_in_a_block_far_back(dev, window, pool, ps):
    """One key (or one block's keys) lines up with the last query many times more than any other.  Just inside the window
    the output IS that key's value; one token further back the key is gone (its block is not complete before the window);
    once its whole block lies before the window the block's mean value comes through; a block far back among dozens is
    found just the same.  In a prompt portion and as a single decoded token."""
    H, G, D = 2, 1, 32
    n = 40 * pool + window + 3                       # dozens of blocks
    last = n - 1
    lo = last - window + 1
    cases = {"inside": lo, "outside": lo - 1 if lo % pool else lo - 2, "far": 3 * pool}      # "outside" avoids a block's last place
    for name, j in cases.items():
        for decode in (False, True):
            def standout(q, k, v, j=j, name=name):
                u = np.zeros(D)
                u[5] = 1.0
                q[0][last] = 40.0 * u
                targets = range(j - j % pool, j - j % pool + pool) if name == "far" else [j]
                for t in targets:
                    k[0][t, 0] = 8.0 * u + 0.01 * k[0][t, 0]
            cuts = [(n - 1,), (1,)] if decode else [(n - 9,), (9,)]
            got, want = _pooled_case(dev, (n,), H, G, D, D, window, pool, ps, torch.float32, cuts, seed=window, standout=standout)
            np.testing.assert_allclose(got[0], want[0], rtol=3e-5, atol=3e-5)
            rng = np.random.default_rng(window)             # the same draws as the case's: its values
            rng.standard_normal((n, H, D)), rng.standard_normal((n, G, D))
            v = torch.from_numpy(rng.standard_normal((n, G, D)).astype(np.float32)).numpy()
            o = got[0][last, 0]
            if name == "inside":
                np.testing.assert_allclose(o, v[j, 0], atol=2e-3)
            elif name == "far":
                b = j // pool
                np.testing.assert_allclose(o, v[b * pool:(b + 1) * pool, 0].mean(0), atol=2e-3)
            else:
                assert np.abs(o - v[j, 0]).max() > 0.3       # the key that would have won is not seen


@pytest.mark.parametrize("heads,dim,vdim", [(3, 8, 20), (1, 64, 64), (5, 6, 7), (2, 130, 33), (80, 16, 16)])
def test_forget_gate_recurrence_through_its_part(dev, heads, dim, vdim):
    """Portions down to one token beside one another, in state rows that were used before; a lower bound near one keeps
    what the first tokens wrote for hundreds of tokens."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import MIXERS
    from sllm_b200.parts.base import LayerCache
    W = 40
    rng = np.random.default_rng(heads * dim)
    K, V = heads * dim, heads * vdim
    w = {"q": rng.standard_normal((K, W)) * 0.3, "f": rng.standard_normal((K, W)) * 0.5, "f.b": rng.standard_normal(K),
         "lower": rng.uniform(0.0, 1.0, K), "v": rng.standard_normal((V, W)) * 0.3, "norm": rng.standard_normal(vdim),
         "o": rng.standard_normal((W, V)) * 0.2}
    w["lower"][::3] = 0.9995                                     # channels that all but never forget
    w = _bf16_exact(w)
    part = MIXERS.build(PartSpec("forget_gate_attention", {"hidden_size": W, "heads": heads, "dim": dim, "vdim": vdim, "eps": 1e-5, "out_scale": 0.7}),
                        dtype=torch.float32, device=dev)
    part.bind(lambda rel: torch.from_numpy(w[rel].astype(np.float32)))
    lens = {0: 131, 1: 40, 2: 3}
    x = {s: rng.standard_normal((n, W)) for s, n in lens.items()}
    state = torch.full((5, heads, dim, vdim), 7.0, dtype=torch.float32, device=dev)       # rows someone used before
    slots = {0: 3, 1: 0, 2: 4}
    for s in slots.values():
        state[s].zero_()                                         # (what the cache manager does at admission)
    cache = LayerCache(state=state, states={"forget_gate": state})
    at, got = {s: 0 for s in lens}, {s: [] for s in lens}
    for cut in [(70, 1, 1), (1, 2, 1), (2, 9, 1), (13, 1, 1), (1, 1, 1), (40, 40, 40), (99, 99, 99)]:
        live = [s for s in lens if at[s] < lens[s]]
        if not live:
            break
        q = [min(cut[s], lens[s] - at[s]) for s in live]
        step = _step(dev, q, [slots[s] for s in live], [at[s] + n for s, n in zip(live, q)])
        term = part.forward(_to(dev)(np.concatenate([x[s][at[s]:at[s] + n] for s, n in zip(live, q)])), step, cache, None)
        y = (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
        r0 = 0
        for s, n in zip(live, q):
            got[s].append(y[r0:r0 + n])
            r0 += n
            at[s] += n
    for s in lens:
        want = 0.7 * plain.recurrent_side(x[s], w, {"heads": heads, "dim": dim, "vdim": vdim}, 1e-5)
        np.testing.assert_allclose(np.concatenate(got[s]), want, rtol=3e-4, atol=3e-4)
    # the long memory is real: without the first 60 tokens the last output differs
    cutoff = 0.7 * plain.recurrent_side(x[0][60:], w, {"heads": heads, "dim": dim, "vdim": vdim}, 1e-5)
    assert np.abs(cutoff[-1] - np.concatenate(got[0])[-1]).max() > 1e-3


@pytest.mark.parametrize("E,top,ff", [(5, 2, 40), (4, 4, 24), (1, 1, 18), (64, 6, 8), (7, 1, 9)])
def test_softmax_router_and_gated_experts(dev, E, top, ff):
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import FEED_FORWARDS
    rng = np.random.default_rng(E * ff)
    W, T = 36, 41
    w = {"router": rng.standard_normal((E, W)) * 0.5}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (rng.standard_normal(s) * 0.5 for s in ((ff, W), (ff, W), (W, ff)))
    w = _bf16_exact(w)
    part = FEED_FORWARDS.build(PartSpec("gated_experts", {"hidden_size": W, "experts": E, "top": top, "expert_ff": ff, "activation": "silu", "scale": 1.7}),
                               dtype=torch.float32, device=dev)
    part.bind(lambda rel: torch.from_numpy(w[rel].astype(np.float32)))
    h = rng.standard_normal((T, W))
    idx, wts = plain.route(h @ w["router"].T, top, 1.7)
    dense, gi, gw = part.route(_to(dev)(h))
    assert (np.sort(gi.cpu().numpy(), -1) == np.sort(idx, -1)).all()
    np.testing.assert_allclose(np.sort(gw.cpu().numpy(), -1), np.sort(wts, -1), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(dense.cpu().numpy().sum(-1), 1.7, rtol=1e-5)
    term = part.forward(_to(dev)(h), None)
    got = (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
    np.testing.assert_allclose(got, plain.experts(h, w, _moe(E, top, ff, 1.7)), rtol=3e-4, atol=3e-4)
    one = part.forward(_to(dev)(h[7:8]), None)                    # a token alone gets what it gets in the batch
    np.testing.assert_allclose((one.sum(0) if one.dim() == 3 else one).cpu().numpy(), got[7:8], rtol=1e-5, atol=3e-5)


def test_attention_side_through_its_part(tmp_path, dev):
    """Projections, the rotation's pairing (channel i with i + dims/2), the factor per head, window, blocks and the sink
    through the part and a cache manager of its own, in portions, against the plain statement."""
    from sllm_b200.cache.manager import CacheManager
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.engine import StepEntry
    from sllm_b200.engine.batch import BatchLayout, context, pack
    from sllm_b200.parts import MIXERS
    W, T = 48, 90
    p = _left(6, 2, 20, 12, 0.3, 11, 4, rot=12, base=200.0, scaling={"factor": 5.0, "low": 1.0, "high": 5.0, "original": 30})
    rng = np.random.default_rng(9)
    w = {"q": rng.standard_normal((120, W)) * 0.4, "k": rng.standard_normal((40, W)) * 0.4, "v": rng.standard_normal((24, W)) * 0.4,
         "temp": rng.uniform(0.5, 2.0, 6), "o": rng.standard_normal((W, 72)) * 0.3}
    w = _bf16_exact(w)
    params = {"hidden_size": W, "heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "scale": 0.3, "window": 11, "pool": 4, "sink": 0.0,
              "out_scale": 1.0, "max_positions": 256, "rotary": {"theta": 200.0, "rotary_dim": 12, "scaling": p["rot"]["scaling"]}}
    part = MIXERS.build(PartSpec("pooled_window_attention", params), dtype=torch.float32, device=dev)
    part.bind(lambda rel: torch.from_numpy(w[rel].astype(np.float32)))
    cm = CacheManager([("own", part.cache_need())], page_size=8, num_pages=[7, 3], max_requests=1)      # the window lets pages go: 7 suffice for 12
    cache = cm.allocate_storage(torch.float32, dev)[0]
    h = rng.standard_normal((T, W))
    got, at = [], 0
    for n in (5, 1, 1, 30, 2, 17, 1, 33):
        e = StepEntry("a", [0] * n, [])
        if at == 0:
            cm.add_request("a")
        cm.reserve("a", at + n)
        lay = BatchLayout(n, 1, 0, [len(t) for t in cm.requests["a"].tables])
        host = np.zeros(lay.total, dtype=np.int32)
        pack(lay, host, cm, [e], [at + n])
        step = context(lay, torch.from_numpy(host).to(dev), 8, [n], [at + n])
        term = part.forward(_to(dev)(h[at:at + n]), step, cache, None)
        got.append((term.sum(0) if term.dim() == 3 else term).cpu().numpy())
        cm.commit("a", at + n)
        at += n
    np.testing.assert_allclose(np.concatenate(got), plain.attention_side(h, w, p, None), rtol=3e-4, atol=3e-4)


# ---- the whole model through the engine: every cutting against the plain implementation ---------------------------

@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_every_cutting_against_plain(tmp_path, dev, which):
    """Whole prompts; most of a prompt and the rest token by token; portions of changing size down to two tokens; up to
    four requests at a time, portions beside single tokens.  The pools hold the trace's peak only and freed pages are
    poisoned, so pages and state slots are used again and a read of a page no longer held would show."""
    from sllm_b200.engine import Engine, build_model
    config, page = CONFIGS[which]
    reqs = _requests(config["vocab"], (70, 37, 100, 1, 45, 64, 23))
    for dtype, d, want, margins in models_for(tmp_path, config, dev, reqs):
        model, _ = build_model(d, dtype, dev)
        for mode in ("whole", "tail_decode", "portions", "mixed"):
            tr = getattr(traces, mode)(reqs)
            eng = Engine(model, page_size=page, num_pages=max(tr.max_tokens // page, 1), max_requests=4, poison_freed=True)
            out = traces.replay_engine(tr, eng)
            compare(tr, out, want, dtype, f"{which}/{dtype}/{mode}", margins)
            eng.cache.check()
            assert not eng.cache.requests and all(g.pool.used_count == 0 for g in eng.cache.groups)
            if mode == "mixed":
                assert eng.cache.reuse_count > 0


def test_stream_after_every_layer_run(tmp_path):
    """The plain statement's stream after each run of a layer (a layer of the loop counts every time) gives, through the
    model's norm and head, the logits of the same weights under a configuration that stops there."""
    d = make_model(tmp_path, ODD)
    cfg, w = plain.load_model(d)
    ids = _requests(ODD["vocab"], (19,))["r0"]
    runs = []
    plain.forward(cfg, w, ids, collect=runs)
    assert len(runs) == 3
    for upto in (1, 2):
        short = dict(cfg, layers=cfg["layers"][:upto])
        x = plain.rms_norm(runs[upto - 1], w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T
        np.testing.assert_allclose(plain.forward(short, w, ids), x, rtol=1e-9, atol=1e-9)
    d = make_model(tmp_path, LOOP_ALL, name="loop")
    cfg, w = plain.load_model(d)
    runs = []
    plain.forward(cfg, w, ids, collect=runs)
    assert len(runs) == 10 and plain.run_order(cfg)[2] == (0, 1)


def test_batch_of_unequal_requests_equals_each_alone(tmp_path, dev):
    from sllm_b200.engine import Engine, StepEntry, build_model
    d = make_model(tmp_path, CONFIG_A)
    reqs = _requests(CONFIG_A["vocab"], (33, 2, 19, 50), seed=8)
    model, _ = build_model(d, "float32", dev)
    alone = {}
    for r, ids in reqs.items():
        eng = Engine(model, page_size=16, num_pages=8, max_requests=2)
        a = eng.step([StepEntry(r, ids[:-1], [len(ids) - 2])])
        b = eng.step([StepEntry(r, ids[-1:], [0])])
        alone[r] = torch.cat([a, b]).cpu().numpy()
    eng = Engine(model, page_size=16, num_pages=16, max_requests=5)
    eng.step([StepEntry("warm", [1, 2, 3], [])])            # takes slot 0 and the first page, then leaves
    eng.finish("warm")
    order = ["r3", "r1", "r0", "r2"]
    a = eng.step([StepEntry(r, reqs[r][:-1], [len(reqs[r]) - 2]) for r in order]).cpu().numpy()
    b = eng.step([StepEntry(r, reqs[r][-1:], [0]) for r in order]).cpu().numpy()
    for i, r in enumerate(order):
        np.testing.assert_allclose(np.stack([a[i], b[i]]), alone[r], rtol=2e-5, atol=2e-5)


def test_a_slot_that_is_used_again_starts_from_nothing(tmp_path, dev):
    """Four state slots, nine requests one after another and side by side: a request that gets a slot and pages another
    one left behind must not see that one's recurrent state, keys or blocks."""
    from sllm_b200.engine import Engine, StepEntry, build_model
    d = make_model(tmp_path, ODD)
    reqs = _requests(ODD["vocab"], (12, 30, 7, 18, 3, 25, 9, 14, 2), seed=17)
    want = plain_logits(d, reqs)
    model, _ = build_model(d, "float32", dev)
    eng = Engine(model, page_size=8, num_pages=16, max_requests=4, poison_freed=True)
    names = list(reqs)
    for a in range(0, len(names), 3):
        group = names[a:a + 3]
        first = eng.step([StepEntry(r, reqs[r][:-1], [len(reqs[r]) - 2]) for r in group]).cpu().numpy()
        last = eng.step([StepEntry(r, reqs[r][-1:], [0]) for r in group]).cpu().numpy()
        for i, r in enumerate(group):
            np.testing.assert_allclose(first[i], want[r][-2], rtol=3e-4, atol=3e-4)
            np.testing.assert_allclose(last[i], want[r][-1], rtol=3e-4, atol=3e-4)
            eng.finish(r)
    assert eng.cache.reuse_count > 0


LONG_MEMORY = {       # blocks far back matter (sharp attention) and the recurrence all but never forgets
    "architecture": "Gerupel", "vocab": 150, "width": 128, "residual_mult": 0.5, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "parallel", "mixer": _mixer(_left(4, 2, 32, 32, 0.2, 24, 6, rot=16, scaling=SCALING), (2, 32, 32), 1.0, 1.0), "mlp": _moe(4, 2, 32, 1.0)},
        {"type": "parallel", "mixer": _mixer(_left(2, 1, 64, 48, 0.15, 36, 12, rot=32), (1, 64, 32), 1.0, 1.0), "mlp": None},
    ],
}


def _sharp(t):
    """Queries many times larger (a softmax that all but picks one key or block), gates whose lower bound is all but one,
    output projections large enough that either mixer's loss shows in the logits."""
    for n in list(t):
        if n.endswith("left.q"):
            t[n] *= 4.0
        if n.endswith("right.lower"):
            t[n] = t[n] * 0 + torch.linspace(0.9, 0.9999, t[n].numel())
        if n.endswith(".o"):
            t[n] *= 2.0


def test_blocks_far_back_page_borders_and_a_long_memory(tmp_path, dev):
    """Sharpened weights (`_sharp`): a prompt of several hundred tokens, cut at and beside page, window and block borders,
    then decoded token by token across more of them; every position wanted."""
    from sllm_b200.engine import Engine, build_model
    config, page = LONG_MEMORY, 16
    reqs = _requests(config["vocab"], (260,), seed=12)
    ids = reqs["r0"]
    for dtype, d, want, margins in models_for(tmp_path, config, dev, reqs, seed=11, edit=_sharp):
        cfg, w = plain.load_model(d)
        cut = plain.forward(cfg, w, ids[150:])              # the memory matters: without the first 150 tokens the end differs
        assert np.abs(cut[-1] - want["r0"][-1]).max() > 0.05
        model, _ = build_model(d, dtype, dev)
        tr = traces.Trace()
        at = 0
        for n in (15, 1, 1, 16, 14, 1, 1, 2, 45, 1, 2, 3, 25):     # up to, onto and over page borders
            tr.step([("r0", at, ids[at:at + n], range(n))])
            at += n
        while at < len(ids):
            tr.step([("r0", at, ids[at:at + 1], [0])], end=["r0"] if at == len(ids) - 1 else [])
            at += 1
        eng = Engine(model, page_size=page, num_pages=tr.max_tokens // page, max_requests=1, poison_freed=True)
        compare(tr, traces.replay_engine(tr, eng), want, dtype, f"far/{dtype}", margins, sharp=True)


def test_long_decoding_from_a_short_prompt(tmp_path, dev):
    """Three tokens of prompt, then 150 tokens one at a time: the states, the pages and the blocks' entries carry
    everything; every step's logits against the plain implementation.  The first tokens of the sequence are wanted too
    (an empty state, a softmax over one key and the sink, no block yet)."""
    from sllm_b200.engine import Engine, build_model
    reqs = _requests(CONFIG_A["vocab"], (153,), seed=42)
    for dtype, d, want, margins in models_for(tmp_path, CONFIG_A, dev, reqs, seed=41):
        model, _ = build_model(d, dtype, dev)
        tr = traces.tail_decode(reqs, tail=150)
        eng = Engine(model, page_size=8, num_pages=tr.max_tokens // 8, max_requests=1)
        compare(tr, traces.replay_engine(tr, eng), want, dtype, f"long/{dtype}", margins)
        tr = traces.Trace()
        tr.step([("r0", 0, reqs["r0"][:1], [0])])
        tr.step([("r0", 1, reqs["r0"][1:2], [0])])
        tr.step([("r0", 2, reqs["r0"][2:5], [0, 1, 2])], end=["r0"])
        eng = Engine(model, page_size=8, num_pages=8, max_requests=1)
        compare(tr, traces.replay_engine(tr, eng), want, dtype, f"first/{dtype}", margins)


def test_greedy_generation_through_the_entry_point(tmp_path, dev):
    """`LLM.generate`: admission, the token budget, prompts in portions, decoding (from captured graphs on the GPU),
    sampling on the device; against greedy decoding with the plain implementation."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine.llm import LLM
    from sllm_b200.sampling import SamplingParams
    d = make_model(tmp_path, CONFIG_A, seed=21)
    cfg, w = plain.load_model(d)
    prompts = list(_requests(CONFIG_A["vocab"], (9, 40, 17, 3, 26), seed=22).values())
    new = 10
    model, _ = build_model(d, "float32", dev)
    llm = LLM(model=model, block_size=16, num_pages=40, max_num_seqs=3, chunk_size=16, max_batch_tokens=48, max_model_len=128)
    res = llm.generate(prompts, SamplingParams(max_new=new))
    for pr, r in zip(prompts, res):
        ids, out = list(pr), []
        for _ in range(new):
            logits = plain.forward(cfg, w, ids)[-1]
            top = np.sort(logits)[-2:]
            out.append(int(np.argmax(logits)))
            ids.append(out[-1])
            if top[1] - top[0] < 1e-3:      # a tie the rounding may break either way: compare up to here
                break
        assert r.ids[:len(out)] == out, (len(pr), r.ids, out)
    llm.engine.cache.check()
    assert not llm.engine.cache.requests


def test_command_line_with_random_weights(tmp_path, capsys, dev, monkeypatch):
    import sllm_b200.engine.llm as llm_mod
    from sllm_b200.serving import main as cli
    recipe = "tiny-gerupel"
    if dev == "cpu":
        import yaml
        real = llm_mod.LLM
        monkeypatch.setattr(llm_mod, "LLM", lambda model_dir, **kw: real(model_dir, **dict(kw, device="cpu")))
        with open(os.path.join(cli.RECIPES_DIR, "tiny-gerupel.yaml")) as f:
            raw = yaml.safe_load(f)
        raw["memory"] = {"kv_device_bytes": 1 << 20}
        recipe = os.path.join(str(tmp_path), "tiny-gerupel.yaml")
        with open(recipe, "w") as f:
            yaml.safe_dump(raw, f)
    assert cli.main([recipe]) == 0
    out = capsys.readouterr().out
    assert "Gerupel: 3 layers" in out
    assert cli.main([recipe, "--mode", "run", "--random-weights", "4", "--prompt-ids", "5,17,3,150,42", "--max-new", "5",
                     "--dtype", "float32", "--log-level", "ERROR"]) == 0
    got = [int(t) for t in capsys.readouterr().out.strip().split(",")]
    assert len(got) == 5 and all(0 <= t < 260 for t in got)


@pytest.mark.gpu
def test_replay_program_on_a_model_folder(tmp_path):
    """bin/trace_run as a user runs it: the model class chosen by config.json, all four cuttings in one trace, four state slots."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    reqs = _requests(CONFIG_B["vocab"], (40, 75, 9, 120, 51), seed=32)
    tr = traces.all_modes(reqs)
    for dtype, d, want, margins in models_for(tmp_path, CONFIG_B, "cuda:0", reqs, seed=31):
        want = traces.tagged(want)
        out_dir = os.path.join(str(tmp_path), f"out_{dtype}")
        out = traces.replay_subprocess(tr, d, dtype, out_dir, 16)
        compare(tr, out, want, dtype, f"replay/{dtype}", margins)
