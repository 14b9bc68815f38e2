"""The Kidolorn design in the engine against the plain numpy statement of it (tests/plain/kidolorn_plain.py).

Every test makes its own small configuration and random weights.  Each body runs twice: with the PyTorch stand-ins
for the kernels on the CPU (the parts, the cache manager, the batching), and on the GPU with the real kernels (marked
``gpu``).  The configurations differ from one another in everything a configuration can say: the order of the three
kinds of mixers, convolutions of one to five taps, key, rotated and value sizes that differ, latents read by one, two
or no later layer, routers that choose one, some or all of their experts, layers without a feed-forward.
"""

import json
import os

import numpy as np
import pytest
import torch

import sllm_b200.models  # noqa: F401  (registers the parts and the architecture)
from tests import traces
from tests.plain import kidolorn_plain as plain


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _decays(n, lo=0.5, hi=0.998):
    return [float(x) for x in 1.0 - (1.0 - lo) * ((1.0 - hi) / (1.0 - lo)) ** (np.arange(n) / max(n - 1, 1))]


CONFIG_A = {          # latents first, read again two layers on; every kind of mixer and of feed-forward; a layer without one
    "architecture": "Kidolorn", "vocab": 310, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 24, 8, 40, 48, 0.2, 1000.0), "mlp": _moe(6, 2, 40, 1.5)},
        {"type": "lightning", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "decay": _decays(3)}, "mlp": _dense(72, 0.8)},
        {"type": "latent_attention", "mixer": _latent(2, 32, 8, 16, 48, 0.15, 1000.0, kv_from=0), "mlp": None},
        {"type": "mingru", "mixer": {"width": 72}, "mlp": _moe(4, 4, 24, 3.0)},
    ],
}
CONFIG_B = {          # latent plus rotated part of 64 on pages of 16: the tensor-core attention forms on the GPU (bfloat16)
    "architecture": "Kidolorn", "vocab": 200, "width": 128, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
    "layers": [
        {"type": "mingru", "mixer": {"width": 160}, "mlp": _dense(192, 1.0)},
        {"type": "lightning", "mixer": {"heads": 2, "dim": 64, "vdim": 64, "decay": [0.9, 0.9995]}, "mlp": _dense(64, 2.0)},
        {"type": "latent_attention", "mixer": _latent(8, 16, 16, 32, 48, 0.18, 10000.0), "mlp": _moe(8, 1, 32, 1.0)},
        {"type": "latent_attention", "mixer": _latent(3, 64, 16, 64, 48, 0.11, 10000.0, kv_from=2), "mlp": _dense(256, 0.5)},
        {"type": "latent_attention", "mixer": _latent(2, 32, 32, 32, 96, 0.12, 500.0), "mlp": _moe(4, 3, 64, 2.0)},
        {"type": "latent_attention", "mixer": _latent(4, 16, 16, 24, 48, 0.2, 10000.0, kv_from=2), "mlp": None},
    ],
}
ODD = {               # sizes that are multiples of nothing; five taps; one head; all experts chosen and one of three
    "architecture": "Kidolorn", "vocab": 77, "width": 50, "norm": {"eps": 1e-4}, "canon": {"taps": 5},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 5, "dim": 6, "vdim": 10, "decay": _decays(5, 0.3, 0.97)}, "mlp": _moe(3, 3, 14, 0.7)},
        {"type": "latent_attention", "mixer": _latent(3, 10, 6, 14, 21, 0.4, 50.0), "mlp": _moe(3, 1, 18, 1.1)},
        {"type": "mingru", "mixer": {"width": 33}, "mlp": None},
        {"type": "latent_attention", "mixer": _latent(1, 12, 6, 9, 21, 0.3, 50.0, kv_from=1), "mlp": _dense(22, 1.3)},
        {"type": "lightning", "mixer": {"heads": 1, "dim": 20, "vdim": 7, "decay": [0.8]}, "mlp": _dense(9, 5.0)},
    ],
}
ONE_TAP = {"architecture": "Kidolorn", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "canon": {"taps": 1},
           "layers": [{"type": "mingru", "mixer": {"width": 64}, "mlp": None},
                      {"type": "latent_attention", "mixer": _latent(2, 16, 2, 16, 30, 0.25, 10.0), "mlp": None}]}
TWO_TAPS = {"architecture": "Kidolorn", "vocab": 120, "width": 72, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
            "layers": [{"type": "lightning", "mixer": {"heads": 4, "dim": 32, "vdim": 16, "decay": _decays(4)}, "mlp": _moe(16, 5, 8, 1.0)},
                       {"type": "mingru", "mixer": {"width": 40}, "mlp": _dense(100, 1.0)}]}
MID = {               # a few hundred channels, no power of two: the products' tensor-core forms at sizes between tiny and real
    "architecture": "Kidolorn", "vocab": 1000, "width": 320, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
    "layers": [
        {"type": "lightning", "mixer": {"heads": 5, "dim": 64, "vdim": 48, "decay": _decays(5, 0.6, 0.9999)}, "mlp": _moe(8, 3, 96, 2.0)},
        {"type": "latent_attention", "mixer": _latent(5, 48, 16, 64, 80, 0.125, 20000.0), "mlp": _dense(768, 1.5)},
        {"type": "mingru", "mixer": {"width": 448}, "mlp": _moe(8, 3, 96, 2.0)},
        {"type": "latent_attention", "mixer": _latent(10, 24, 16, 32, 80, 0.16, 20000.0, kv_from=1), "mlp": _dense(768, 1.5)},
        {"type": "mingru", "mixer": {"width": 448}, "mlp": None},
        {"type": "lightning", "mixer": {"heads": 5, "dim": 64, "vdim": 48, "decay": _decays(5, 0.6, 0.9999)}, "mlp": _dense(512, 1.0)},
    ],
}
CONFIGS = {"A": (CONFIG_A, 16), "B": (CONFIG_B, 16), "odd": (ODD, 8), "one_tap": (ONE_TAP, 4), "two_taps": (TWO_TAPS, 32), "mid": (MID, 16)}


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
    """{request: logits}; ``margins`` (a dict) receives per request the smallest relative gap, per position, between the last
    chosen expert's logit and the best one left out, over all routers."""
    cfg, w = plain.load_model(d)
    out = {}
    for r, ids in reqs.items():
        m = []
        out[r] = plain.forward(ids, cfg, w, margins=m).astype(np.float32)
        if margins is not None:
            margins[r] = np.min(np.stack(m), axis=0) if m else np.full(len(ids), np.inf)
    return out


def dtypes_on(dev):
    return ("float32",) if dev == "cpu" else ("float32", "bfloat16")


def models_for(tmp_path, config, dev, reqs, seed=5, edit=None):
    """(dtype, model folder, plain logits, routers' margins) for every dtype the device runs."""
    for dtype in dtypes_on(dev):
        d = make_model(tmp_path, config, seed=seed, name=f"m_{dtype}", edit=edit)
        margins = {}
        yield dtype, d, plain_logits(d, reqs, margins), margins


CLOSE_CALL = 0.04


def compare(tr, out, want, dtype, what, margins=None):
    """float32: every logit to 3e-4.  bfloat16: the difference of a row (mean taken off, root mean square over the
    vocabulary) relative to the row's own spread is rounding's: under 4 % for 19 rows in 20 and under 15 % for every
    row.  bfloat16 rounding moves a router's logits by a per cent or so of their size; a token whose last chosen expert
    and first left-out one lie closer than that may go to the other one, which changes its whole feed-forward term and
    is no fault: such rows (``margins`` under `CLOSE_CALL`) are left out of the bfloat16 comparison.  The float32 runs
    compare every row."""
    if dtype == "float32":
        return traces.compare(tr, out, want, what=what, rtol=3e-4, atol=3e-4)
    errs, skipped = [], 0
    for s in tr.steps:
        for row, (req, pos) in enumerate(s["expect"]):
            if margins is not None and margins[req.split(".")[-1]][pos] < CLOSE_CALL:
                skipped += 1
                continue
            ref, got = want[req][pos], out[s["step"]][row]
            d, r = got - ref, ref - ref.mean()
            e = float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((r ** 2).mean()))
            assert e < 0.15, f"{what}: step {s['step']}, request {req!r}, position {pos}: relative difference {e:.3g}"
            errs.append(e)
    assert skipped <= len(errs), f"{what}: {skipped} rows left out for close calls, {len(errs)} compared"
    assert np.quantile(errs, 0.95) < 0.04, f"{what}: 95th percentile of the rows' relative difference {np.quantile(errs, 0.95):.3g}"


def _requests(vocab, lengths, seed=3):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, n).tolist() for i, n in enumerate(lengths)}


def _to(dev):
    return lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).contiguous()


def _bf16_exact(w):
    """The arrays rounded to what bfloat16 holds (a float32 part keeps such weights exactly; a float64 plain function too)."""
    return {n: torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64) for n, a in w.items()}


def _step(dev, q_lens, slots, ctx_lens=None, group=None):
    """A batch description by hand: portions of ``q_lens`` tokens that end at ``ctx_lens`` (default: start at 0)."""
    from sllm_b200.parts import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ctx_lens = list(ctx_lens or q_lens)
    starts = np.concatenate([[0], np.cumsum(q_lens)])
    pos = np.concatenate([np.arange(c - q, c) for q, c in zip(q_lens, ctx_lens)])
    return StepContext(num_tokens=int(starts[-1]), num_seqs=len(q_lens), token_ids=i32([0] * int(starts[-1])), positions=i32(pos.tolist()),
                       seq_of_token=i32(np.repeat(np.arange(len(q_lens)), q_lens).tolist()), q_start=i32(starts.tolist()),
                       ctx_len=i32(ctx_lens), state_slots=i32(slots), logit_rows=i32([]), groups=[group] if group else [],
                       q_lens=list(q_lens), ctx_lens=ctx_lens, max_q_len=max(q_lens), max_ctx_len=max(ctx_lens))


def _portions(dev, lens, slots, cuts, run):
    """Feed requests of ``lens`` tokens side by side in portions ``cuts``; ``run(rows by request, step) -> [T, ...]``."""
    at, got = {s: 0 for s in lens}, {s: [] for s in lens}
    for cut in cuts:
        live = [s for s in lens if at[s] < lens[s]]
        if not live:
            break
        q = [min(cut[s], lens[s] - at[s]) for s in live]
        y = run([(s, at[s], at[s] + n) for s, n in zip(live, q)], _step(dev, q, [slots[s] for s in live], [at[s] + n for s, n in zip(live, q)]))
        r0 = 0
        for s, n in zip(live, q):
            got[s].append(y[r0:r0 + n])
            r0 += n
            at[s] += n
    assert all(at[s] == lens[s] for s in lens)
    return {s: np.concatenate(got[s]) for s in lens}


CUTS = [(70, 1), (1, 2), (2, 9), (13, 1), (1, 1), (40, 40)]


# ---- configuration, plan, weights ---------------------------------------------------------------------------

def test_config_plan_and_cache_needs():
    from sllm_b200.config import ConfigError, architecture_of
    from sllm_b200.models.causal_lm import CausalLM
    from sllm_b200.parts import PagedKV, SlotState
    arch = architecture_of(CONFIG_A)
    cfg = arch.config_cls.from_dict(CONFIG_A)
    assert cfg.to_dict() == CONFIG_A
    p = arch.plan(cfg)
    assert len(p.layers) == 4 and [e.layer for e in p.run_list] == [0, 1, 2, 3] and p.position is None
    assert [e.cache_from for e in p.run_list] == [None, None, 0, None]
    assert "ffn" not in p.layers[2].parts and "ffn_conv" not in p.layers[2].parts and "mixer_conv" in p.layers[2].parts
    m = CausalLM(p, dtype=torch.float32, device="cpu")
    needs = m.cache_needs()
    conv = lambda name: SlotState((96, 2), name)
    assert needs[0] == ("own", (PagedKV(1, 56, None, values=False), conv("conv_mixer"), conv("conv_ffn")))
    assert needs[1] == ("own", (SlotState((3, 16, 24), "lightning"), conv("conv_mixer"), conv("conv_ffn")))
    assert needs[2] == ("borrow", 0, (conv("conv_mixer"),))            # the pages are layer 0's; its convolution's inputs are its own
    assert needs[3] == ("own", (SlotState((72,), "mingru"), conv("conv_mixer"), conv("conv_ffn")))
    names = {s.name for s in m.tensor_specs()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.canon1", "l0.canon2", "l0.mix.dkv",
            "l0.mix.dkv.norm", "l0.mix.sink", "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l0.mlp.e5.down", "l0.mlp.router", "l1.mix.norm",
            "l1.mlp.gate.b", "l1.mlp.down.b", "l2.mix.q", "l2.mix.sink", "l3.mix.z.b", "l3.mix.x.b", "l3.mix.o"} <= names
    assert not any(n.startswith(("l2.mlp", "l2.norm2", "l2.canon2", "l2.mix.dkv")) or n.endswith(("mix.g.b", "e0.gate.b")) for n in names)
    shapes = {s.name: tuple(s.shape) for s in m.tensor_specs()}
    assert shapes["l0.norm1"] == () and shapes["l0.canon1"] == (96, 3) and shapes["l0.mix.q"] == (4 * 32, 96) and shapes["l0.mix.dkv"] == (56, 96)
    assert shapes["l2.mix.uk"] == (2 * 32, 48) and shapes["l2.mix.uv"] == (2 * 16, 48) and shapes["l2.mix.g"] == (2 * 16, 96)

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
    for bad in (edited(("layers", 0, "mlp", "router", "top"), 7),                 # more than there are experts
                edited(("layers", 1, "mixer", "decay"), [0.5, 0.6]),              # one decay per head
                edited(("layers", 2, "mixer", "kv_from"), 1),                     # layer 1 holds no latents
                edited(("layers", 2, "mixer", "kv_from"), 2),                     # nor does a layer lend to itself
                edited(("layers", 2, "mixer", "kv_rank"), 40),                    # the lender's latents have another size
                edited(("layers", 0, "type"), "other"), edited(("layers", 1, "mlp", "kind"), "other"),
                edited(("norm",), None), edited(("layers",), []), edited(("layers", 3, "mixer", "width"), None)):
        with pytest.raises(ConfigError):
            arch.config_cls.from_dict(bad)


def test_a_lender_of_latents_may_not_borrow():
    from sllm_b200.config import ConfigError, architecture_of
    c = json.loads(json.dumps(CONFIG_B))
    c["layers"][5]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError):
        architecture_of(c).config_cls.from_dict(c)


# ---- each mechanism alone: an operation or a part against the plain function ------------------------------------------

@pytest.mark.parametrize("W", [50, 96, 1000, 1500, 3000, 4500])     # the kernel keeps rows of up to 1,024, 2,048 and 4,096 channels in registers
def test_norm_with_one_number_before_and_after_a_sublayer(dev, W):
    """The sublayer's term (whole, and as a stack of partial sums) is normed with one number, joins the stream, and the
    stream is normed with another number for the next reader; each half alone too."""
    import sllm_b200.ops as ops
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import NORMS
    rng = np.random.default_rng(W)
    T, eps = 7, 1e-3
    x, y = rng.standard_normal((T, W)) * 3, rng.standard_normal((3, T, W)) * 0.02        # (a small term: eps counts)
    to = _to(dev)
    norms = {}
    for name, g in (("post", -1.7), ("pre", 0.6)):
        norms[name] = NORMS.build(PartSpec("scalar_rmsnorm", {"size": W, "eps": eps}), dtype=torch.float32, device=dev)
        norms[name].bind(lambda rel, g=g: torch.tensor(g))
        assert tuple(norms[name].weight.shape) == (W,)
    post, pre = norms["post"], norms["pre"]
    want_stream = x + plain.norm_scalar(y.sum(0), -1.7, eps)
    for term in (to(y.sum(0)), to(y)):
        stream = to(x)
        h = ops.post_add_norm(stream, term, post.weight, post.eps, pre.weight, pre.eps)
        np.testing.assert_allclose(stream.cpu().numpy(), want_stream, rtol=2e-5, atol=2e-5)
        np.testing.assert_allclose(h.cpu().numpy(), plain.norm_scalar(want_stream, 0.6, eps), rtol=2e-5, atol=2e-5)
    stream = to(x)
    assert ops.post_add_norm(stream, to(y), post.weight, post.eps, None, 0.0) is None
    np.testing.assert_allclose(stream.cpu().numpy(), want_stream, rtol=2e-5, atol=2e-5)
    stream = to(x)
    h = pre.add_norm(stream, None)
    np.testing.assert_allclose(h.cpu().numpy(), plain.norm_scalar(x, 0.6, eps), rtol=2e-5, atol=2e-5)
    np.testing.assert_array_equal(stream.cpu().numpy(), x.astype(np.float32))


@pytest.mark.parametrize("C,taps", [(10, 2), (70, 3), (300, 4), (33, 5), (8, 1), (12, 2), (64, 3), (516, 4), (16, 6)])
def test_input_convolution_across_portions_and_slots(dev, C, taps):
    """h + conv(h) for two requests side by side in portions down to one token (shorter than the taps), continuing from
    their state rows, one of which held another request's inputs before (zeroed on admission by the cache manager; here
    by hand); a third row stays untouched."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import SHIFTS
    rng = np.random.default_rng(C)
    lens = {0: 29, 1: 17}
    xs = {s: rng.standard_normal((n, C)) for s, n in lens.items()}
    w = rng.standard_normal((C, taps))
    conv = SHIFTS.build(PartSpec("input_conv", {"size": C, "taps": taps}), dtype=torch.float32, device=dev)
    conv.bind(lambda rel: torch.from_numpy(w.astype(np.float32)))
    need = conv.state("s")
    assert (need is None) == (taps == 1)
    state = torch.zeros((3,) + tuple(need.shape), dtype=torch.float32, device=dev) if need else None
    slots = {0: 2, 1: 0}
    to = _to(dev)
    got = _portions(dev, lens, slots, [(1, 2), (1, 1), (2, 1), (9, 6), (1, 1), (3, 2), (20, 20)],
                    lambda rows, step: conv(to(np.concatenate([xs[s][a:b] for s, a, b in rows])), state, step).cpu().numpy())
    for s in lens:
        np.testing.assert_allclose(got[s], plain.input_convolution(xs[s], w), rtol=2e-5, atol=2e-5)
        if taps > 1:
            np.testing.assert_allclose(state[slots[s]].cpu().numpy(), xs[s][-(taps - 1):].T, rtol=1e-6)
    assert taps == 1 or float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("W,taps", [(50, 3), (96, 4), (1000, 2), (24, 1), (40, 6), (1500, 4), (3000, 3), (4500, 2)])
def test_norm_and_convolution_in_one_kernel_for_single_tokens(dev, W, taps):
    """A block's read of the stream where every request brings one token: the term of the sublayer before joins the stream
    behind its norm, the stream is normed, and h + conv(h) comes back, all in one call; three requests decode side by side for
    a while, one leaves, and a new one takes its state row (zeroed by hand, as the cache manager does on admission).  A
    portion of several tokens in between goes the two-kernel way through the same block and must continue the same state."""
    import sllm_b200.ops as ops
    rng = np.random.default_rng(W + taps)
    eps, g_post, g_pre = 1e-5, 0.7, -1.3
    wconv = rng.standard_normal((W, taps))
    lens = {"a": 14, "b": 9, "c": 11}
    x = {r: rng.standard_normal((n, W)) * 3.0 for r, n in lens.items()}                # the stream before the term
    y = {r: rng.standard_normal((2, n, W)) for r, n in lens.items()}                   # the term as two partial sums
    want, stream_want = {}, {}
    for r in lens:
        stream_want[r] = x[r] + plain.norm_scalar(y[r].sum(0), g_post, eps)
        want[r] = plain.input_convolution(plain.norm_scalar(stream_want[r], g_pre, eps), wconv)
    to = _to(dev)
    gain = lambda v: torch.full((W,), v, dtype=torch.float32, device=dev)
    wt = to(wconv)
    state = torch.full((3, W, taps - 1), 7.0, dtype=torch.float32, device=dev) if taps > 1 else None
    slot = {"a": 1, "b": 0, "c": 1}                                                    # c takes a's row when a has left
    got = {r: [] for r in lens}

    def run(live, n):
        st = _step(dev, [n[r] for r in live], [slot[r] for r in live])
        at = {r: len(got[r]) for r in live}
        stream = to(np.concatenate([x[r][at[r]:at[r] + n[r]] for r in live]))
        term = to(np.concatenate([y[r][:, at[r]:at[r] + n[r]] for r in live], axis=1))
        if all(n[r] == 1 for r in live):
            out = ops.post_add_norm_conv(stream, term, gain(g_post), eps, gain(g_pre), eps, wt, state, st, torch.float32)
        else:
            h = ops.post_add_norm(stream, term, gain(g_post), eps, gain(g_pre), eps, torch.float32)
            out = ops.short_conv_add(h, wt, state, st, torch.float32)
        out, stream = out.cpu().numpy(), stream.cpu().numpy()
        r0 = 0
        for r in live:
            np.testing.assert_allclose(stream[r0:r0 + n[r]], stream_want[r][at[r]:at[r] + n[r]], rtol=2e-5, atol=2e-5)
            got[r] += list(out[r0:r0 + n[r]])
            r0 += n[r]
    if state is not None:
        state[[0, 1]] = 0.0
    for _ in range(4):
        run(["a", "b"], {"a": 1, "b": 1})
    run(["b", "a"], {"a": 3, "b": 1})                                                  # a portion beside a single token
    while len(got["a"]) < lens["a"]:
        run(["a", "b"] if len(got["b"]) < lens["b"] else ["a"], {"a": 1, "b": 1})
    if state is not None:
        state[1] = 0.0
    while len(got["c"]) < lens["c"]:
        run(["c"], {"c": 1})
    for r in lens:
        np.testing.assert_allclose(np.stack(got[r]), want[r], rtol=3e-5, atol=3e-5)
    if state is not None:
        assert float(state[2].min()) == 7.0 and float(state[2].max()) == 7.0
        np.testing.assert_allclose(state[1].cpu().numpy(), plain.norm_scalar(stream_want["c"], g_pre, eps)[-(taps - 1):].T, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("C", [33, 72, 160, 1])
def test_element_wise_recurrence_in_portions_and_slots(dev, C):
    """The mixer through its part: two requests in portions down to one token against the whole sequences through the
    plain function.  A portion of 70 tokens is cut into runs that the kernel's warps walk side by side; biases push some
    candidates onto each branch and some gates to where the state all but stays."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import MIXERS, LayerCache
    rng = np.random.default_rng(C)
    W = 40
    w = _bf16_exact({"m.z": rng.standard_normal((C, W)) * 0.4, "m.z.b": rng.standard_normal(C) * 2 - 3.0, "m.x": rng.standard_normal((C, W)) * 0.5,
                     "m.x.b": rng.standard_normal(C), "m.g": rng.standard_normal((C, W)) * 0.3, "m.o": rng.standard_normal((W, C)) * 0.3})
    mixer = MIXERS.build(PartSpec("mingru", {"hidden_size": W, "width": C}), dtype=torch.float32, device=dev)
    mixer.bind(lambda rel: torch.from_numpy(w["m." + rel].astype(np.float32)))
    lens, slots = {0: 110, 1: 21}, {0: 2, 1: 0}
    xs = {s: rng.standard_normal((n, W)) for s, n in lens.items()}
    cache = LayerCache(states={"mingru": torch.zeros((3, C), dtype=torch.float32, device=dev)})
    cache.state = cache.states["mingru"]
    to = _to(dev)

    def run(rows, step):
        term = mixer.forward(to(np.concatenate([xs[s][a:b] for s, a, b in rows])), step, cache, None)
        return (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
    got = _portions(dev, lens, slots, CUTS, run)
    for s in lens:
        np.testing.assert_allclose(got[s], plain.mingru(xs[s], w, "m.", {"width": C}), rtol=3e-4, atol=3e-4)
    assert float(cache.states["mingru"][1].abs().max()) == 0.0
    assert float(cache.states["mingru"][2].abs().max()) > 0.0


@pytest.mark.parametrize("C,n,more", [(44, 600, 0), (8, 257, 1), (132, 1100, 3), (30, 300, 0)])
def test_element_wise_recurrence_and_convolution_over_a_long_portion(dev, C, n, more):
    """Portions of hundreds of tokens take other forms of both kernels (many short runs of eight channels; a run of tokens a
    thread): one request's long portion, alone or beside requests that bring a token each, then a second portion that goes on
    from the state rows, against the plain functions over the whole sequence."""
    import sllm_b200.ops as ops
    rng = np.random.default_rng(C + n)
    taps = 4
    tail = 9
    lens = [n + tail] + [2] * more
    proj = [rng.standard_normal((m, 3 * C)) * np.array([1.0] * C + [1.5] * C + [1.0] * C) + np.array([-2.0] * C + [0.0] * (2 * C)) for m in lens]
    wconv = rng.standard_normal((C, taps))
    to = _to(dev)
    state = torch.zeros((more + 2, C), dtype=torch.float32, device=dev)
    cstate = torch.zeros((more + 2, C, taps - 1), dtype=torch.float32, device=dev)
    slots = list(range(more, -1, -1))                                                 # the long request sits in the last row used
    outs, convs = [[] for _ in lens], [[] for _ in lens]
    at = [0] * len(lens)
    for q in ([n] + [1] * more, [tail] + [1] * more):
        step = _step(dev, q, slots, [a + b for a, b in zip(at, q)])
        rows = np.concatenate([proj[i][at[i]:at[i] + q[i]] for i in range(len(lens))])
        y = ops.mingru_scan(to(rows), (0, C, 2 * C), state, step, C, torch.float32).cpu().numpy()
        z = ops.short_conv_add(to(rows[:, :C]), to(wconv), cstate, step, torch.float32).cpu().numpy()
        r0 = 0
        for i in range(len(lens)):
            outs[i].append(y[r0:r0 + q[i]])
            convs[i].append(z[r0:r0 + q[i]])
            r0 += q[i]
            at[i] += q[i]
    for i, p in enumerate(proj):
        zg = 1.0 / (1.0 + np.exp(-p[:, :C]))
        cand = plain.mingru_candidate(p[:, C:2 * C])
        S, want = np.zeros(C), []
        for t in range(len(p)):
            S = (1.0 - zg[t]) * S + zg[t] * cand[t]
            g = p[t, 2 * C:]
            want.append(S * g / (1.0 + np.exp(-g)))
        np.testing.assert_allclose(np.concatenate(outs[i]), np.stack(want), rtol=3e-5, atol=3e-5)
        np.testing.assert_allclose(np.concatenate(convs[i]), plain.input_convolution(p[:, :C], wconv), rtol=3e-5, atol=3e-5)
        np.testing.assert_allclose(state[slots[i]].cpu().numpy(), S, rtol=3e-5, atol=3e-5)
    assert float(state[more + 1].abs().max()) == 0.0 and float(cstate[more + 1].abs().max()) == 0.0


def test_candidate_of_the_recurrence_has_two_branches():
    u = np.array([-30.0, -1.0, -1e-9, 0.0, 1e-9, 2.0])
    c = plain.mingru_candidate(u)
    np.testing.assert_allclose(c, [1 / (1 + np.exp(30.0)), 1 / (1 + np.e), 0.5, 0.5, 0.5, 2.5], rtol=1e-6)
    assert (np.diff(c) >= 0).all()                      # continuous and rising through zero


@pytest.mark.parametrize("heads,dk,dv", [(1, 64, 64), (3, 16, 24), (5, 6, 10), (2, 130, 12), (90, 16, 16), (4, 32, 16), (2, 128, 128), (1, 256, 80), (3, 96, 160)])
def test_linear_attention_with_a_fixed_decay_in_portions_and_slots(dev, heads, dk, dv):
    """S <- decay_h S + k v^T through the part's own `mix` and output projection.  The last head all but never forgets
    (0.9999) and the first forgets within a few tokens; the heads' outputs share ONE root mean square."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import MIXERS, LayerCache
    rng = np.random.default_rng(dk + heads)
    W, eps = 40, 1e-5
    K, V = heads * dk, heads * dv
    decay = _decays(heads, 0.2, 0.9999) if heads > 1 else [0.97]
    w = _bf16_exact({"m.q": rng.standard_normal((K, W)) * 0.3, "m.k": rng.standard_normal((K, W)) * 0.3, "m.v": rng.standard_normal((V, W)) * 0.3,
                     "m.g": rng.standard_normal((V, W)) * 0.3, "m.o": rng.standard_normal((W, V)) * 0.2, "m.norm": 1 + 0.3 * rng.standard_normal(V)})
    mixer = MIXERS.build(PartSpec("decay_linear_attention", {"hidden_size": W, "heads": heads, "dim": dk, "vdim": dv, "decay": decay, "eps": eps}),
                         dtype=torch.float32, device=dev)
    mixer.bind(lambda rel: torch.from_numpy(w["m." + rel].astype(np.float32)))
    lens, slots = {0: 110, 1: 21}, {0: 1, 1: 2}
    xs = {s: rng.standard_normal((n, W)) for s, n in lens.items()}
    m = {"heads": heads, "dim": dk, "vdim": dv, "decay": [float(np.float32(d)) for d in decay]}
    want = {s: plain.lightning(x, w, "m.", m, eps) for s, x in xs.items()}
    cache = LayerCache(states={"lightning": torch.zeros((3, heads, dk, dv), dtype=torch.float32, device=dev)})
    to = _to(dev)

    def run(rows, step):
        term = mixer.forward(to(np.concatenate([xs[s][a:b] for s, a, b in rows])), step, cache, None)
        return (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
    got = _portions(dev, lens, slots, CUTS, run)
    for s in lens:
        np.testing.assert_allclose(got[s], want[s], rtol=5e-4, atol=5e-4)
    assert float(cache.states["lightning"][0].abs().max()) == 0.0


def test_rotation_pairs_a_channel_with_the_one_half_the_dims_on(dev):
    """The table the parts build against the plain frequencies; `rope_cols_` writes each head's rotated columns into a
    slice of wider rows and zeroes what lies behind."""
    import sllm_b200.ops as ops
    from sllm_b200.parts.side_by_side import rotary_for
    rng = np.random.default_rng(4)
    for base, dims, n, H in ((10000.0, 16, 16, 3), (50.0, 6, 6, 1), (500.0, 32, 32, 2), (10.0, 2, 2, 5), (1000.0, 8, 12, 2)):
        rot = {"base": base, "dims": dims}
        table = rotary_for({"theta": base, "rotary_dim": dims, "max_positions": 3000}, torch.float32, dev).table
        f = plain.rotary_frequencies(rot)
        pos = np.array([0, 1, 2, 77, 2999, 1023, 1024])
        np.testing.assert_allclose(table[torch.from_numpy(pos).to(dev), 0].cpu().numpy(), np.cos(pos[:, None] * f[None]), rtol=0, atol=2e-7)
        np.testing.assert_allclose(table[torch.from_numpy(pos).to(dev), 1].cpu().numpy(), np.sin(pos[:, None] * f[None]), rtol=0, atol=2e-7)
        T, xoff, xstride, ooff, ostride = len(pos), 5, n + 9, 11, 11 + n + 3
        x = rng.standard_normal((T, xoff + H * xstride + 2))
        out = torch.full((T, H * ostride), 7.0, dtype=torch.float32, device=dev)
        ops.rope_cols_(out, ooff, ostride, _to(dev)(x), xoff, xstride, n, dims, torch.from_numpy(pos.astype(np.int32)).to(dev), table, H)
        got = out.cpu().numpy().reshape(T, H, ostride)
        src = np.stack([x[:, xoff + h * xstride:xoff + h * xstride + n] for h in range(H)], axis=1)
        np.testing.assert_allclose(got[..., ooff:ooff + n], plain.rotate(src, pos, rot), rtol=2e-5, atol=2e-5)
        assert (got[..., :ooff] == 7.0).all() and not got[..., ooff + n:].any()


def _paged(dev, D, ps, lens, rng, spare=3):
    """A cache of one key-and-value head filled with random rows for requests of ``lens`` tokens on scattered pages."""
    from sllm_b200.parts import GroupView
    per = [-(-n // ps) for n in lens]
    order = rng.permutation(sum(per) + spare)
    tables = np.full((len(lens), max(per) + 1), -1, dtype=np.int32)
    at = 0
    for s, n in enumerate(per):
        tables[s, :n] = order[at:at + n]
        at += n
    k = rng.standard_normal((sum(per) + spare, 1, ps, D)).astype(np.float32)
    g = GroupView(ps, torch.from_numpy(tables).to(dev), torch.zeros(1, dtype=torch.int32, device=dev))
    return k, tables, g


@pytest.mark.parametrize("D,ps,dtype,nq", [(27, 4, "float32", 3), (64, 16, "bfloat16", 4), (64, 16, "bfloat16", 24), (128, 32, "bfloat16", 6),
                                           (32, 8, "bfloat16", 2), (56, 16, "float32", 4), (16, 16, "bfloat16", 1), (128, 64, "bfloat16", 16)])
def test_softmax_with_a_sink_over_keys_near_and_far(dev, D, ps, dtype, nq):
    """Many query heads over ONE cached head that is key and value at once, hundreds of tokens into a request, as single
    decoded tokens and as prompt portions that start and end beside page borders.  For every query one key is made to
    stand out in its first head: the sequence's first token, the one a page back, the query's own.  Head 0's sink is so
    large that it takes most of the weight, head 1's so small that it takes none; the sink has no value, so it only
    shrinks the output."""
    import sllm_b200.ops as ops
    if dev == "cpu" and dtype != "float32":
        pytest.skip("the stand-ins are float32")
    rng = np.random.default_rng(D + nq)
    scale = 0.3
    cases = [(1, 1), (1, 2), (1, 700), (1, 3 * ps), (1, 3 * ps + 1), (2, 2), (5, 5), (2, 2 * ps + 1), (ps + 3, 4 * ps + 2), (3, 333), (150, 150),
             (130, 400), (1, 64), (1, 65)]
    q_lens, ctx = [c[0] for c in cases], [c[1] for c in cases]
    k, tables, g = _paged(dev, D, ps, ctx, rng)
    T = sum(q_lens)
    q = rng.standard_normal((T, nq, D)).astype(np.float32)
    step = _step(dev, q_lens, list(range(len(cases))), ctx, g)
    pos, seq = step.positions.cpu().numpy(), step.seq_of_token.cpu().numpy()
    for t in range(T):
        j = (0, max(pos[t] - ps, 0), pos[t])[t % 3]
        k[tables[seq[t], j // ps], 0, j % ps] = q[t, 0] * (5.0 / np.sqrt(D) * 4)
    sink = rng.standard_normal(nq).astype(np.float32)
    sink[0] = 9.0
    if nq > 1:
        sink[1] = -30.0
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    qd, kd = (torch.from_numpy(a).to(dev).to(td).contiguous() for a in (q.reshape(T, nq * D), k))
    sk = torch.from_numpy(sink).to(dev)
    got = ops.paged_attention(qd, kd, kd, step, 0, nq, 1, D, scale, None, sink=sk).float().cpu().numpy().reshape(T, nq, D)
    plain_got = ops.paged_attention(qd, kd, kd, step, 0, nq, 1, D, scale, None).float().cpu().numpy().reshape(T, nq, D)
    qf, kf = qd.float().cpu().numpy().reshape(T, nq, D).astype(np.float64), kd.float().cpu().numpy().astype(np.float64)
    tol = 3e-5 if dtype == "float32" else 3e-2
    for t in range(T):
        js = np.arange(pos[t] + 1)
        kk = kf[tables[seq[t], js // ps], 0, js % ps]
        for h in range(nq):
            s = kk @ qf[t, h] * scale
            mx = max(s.max(), sink[h])
            e = np.exp(s - mx)
            np.testing.assert_allclose(got[t, h], (e / (e.sum() + np.exp(sink[h] - mx))) @ kk, rtol=tol, atol=tol,
                                       err_msg=f"token {t} (position {pos[t]}), head {h}, with sink")
            np.testing.assert_allclose(plain_got[t, h], (e / e.sum()) @ kk, rtol=tol, atol=tol, err_msg=f"token {t} (position {pos[t]}), head {h}")


@pytest.mark.parametrize("H,dk,dr,dv,rank,H2,dk2,dv2,ps,dtype", [
    (4, 24, 8, 40, 48, 2, 32, 16, 4, "float32"), (3, 10, 6, 14, 21, 1, 12, 9, 8, "float32"), (8, 16, 16, 32, 48, 3, 64, 64, 16, "bfloat16"),
    (2, 32, 32, 32, 96, 5, 8, 24, 16, "bfloat16"), (1, 16, 2, 16, 30, 2, 16, 8, 16, "float32"), (2, 128, 64, 128, 192, 2, 64, 64, 16, "bfloat16"),
    (2, 16, 32, 24, 288, 1, 24, 16, 16, "float32"), (2, 32, 64, 32, 512, 2, 16, 16, 16, "bfloat16")])      # cached rows beyond 256 channels
def test_latent_attention_and_a_second_layer_on_the_same_latents(dev, H, dk, dr, dv, rank, H2, dk2, dv2, ps, dtype):
    """The whole mixer through its part: the latent's norm, the rotated key part that all heads share, queries carried into
    the latent space, the sink, the gate on every output channel; then a second mixer without a down-projection that reads
    what the first one cached, with heads, key and value sizes, scale and sinks of its own.  Two requests in portions
    down to one token on scattered pages."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import MIXERS, GroupView, LayerCache
    if dev == "cpu" and dtype != "float32":
        pytest.skip("the stand-ins are float32")
    rng = np.random.default_rng(rank + H)
    W, eps, base = 72, 1e-5, 300.0
    td = torch.float32 if dtype == "float32" else torch.bfloat16

    def weights(H, dk, dv, own):
        w = {"m.q": rng.standard_normal((H * (dk + dr), W)) * 0.4, "m.uk": rng.standard_normal((H * dk, rank)) * 0.3,
             "m.uv": rng.standard_normal((H * dv, rank)) * 0.3, "m.sink": rng.standard_normal(H) * 2.0, "m.g": rng.standard_normal((H * dv, W)) * 0.3,
             "m.o": rng.standard_normal((W, H * dv)) * 0.2}
        if own:
            w.update({"m.dkv": rng.standard_normal((rank + dr, W)) * 0.4, "m.dkv.norm": 1 + 0.3 * rng.standard_normal(rank)})
        return _bf16_exact(w)

    def build(H, dk, dv, scale, w, shared):
        m = MIXERS.build(PartSpec("latent_attention", {
            "hidden_size": W, "heads": H, "dim": dk, "vdim": dv, "kv_rank": rank, "scale": scale, "eps": eps, "gate": "element", "sink": True,
            "rot_dim": dr, "shared_kv": shared, "rotary": {"theta": base, "rotary_dim": dr, "max_positions": 512}}), dtype=td, device=dev)
        m.bind(lambda rel: torch.from_numpy(w["m." + rel].astype(np.float32)))
        return m
    w1, w2 = weights(H, dk, dv, True), weights(H2, dk2, dv2, False)
    # scales that leave the scores a spread of about 3 and 1.5 (what the weights above give a score before it is scaled)
    spread = lambda dk: 0.4 * np.sqrt(W) * np.sqrt(dk * 0.09 * rank + dr * 0.16 * W)
    sc1, sc2 = float(np.float32(3.0 / spread(dk))), float(np.float32(1.5 / spread(dk2)))
    first, second = build(H, dk, dv, sc1, w1, False), build(H2, dk2, dv2, sc2, w2, True)
    assert first.cache_need() == second.cache_need() and first.cache_need().head_dim >= rank + dr
    lens, slots = {0: 110, 1: 37}, {0: 0, 1: 1}
    xs = {s: _bf16_exact({"x": rng.standard_normal((n, W))})["x"] for s, n in lens.items()}
    m1 = {"heads": H, "dim": dk, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": sc1, "rot": {"base": base, "dims": dr}}
    m2 = dict(m1, heads=H2, dim=dk2, vdim=dv2, scale=sc2)
    want1, want2 = {}, {}
    for s, x in xs.items():
        lat = plain.latent_parts(x, w1, "m.", m1, eps, np.arange(len(x)))
        want1[s] = plain.latent_attention(x, w1, "m.", m1, eps, np.arange(len(x)), lat)
        want2[s] = plain.latent_attention(x, w2, "m.", m2, eps, np.arange(len(x)), lat)
    D = first.cache_need().head_dim
    _, tables, _ = _paged(dev, D, ps, list(lens.values()), rng)
    kc = torch.full((int(tables.max()) + 1, 1, ps, D), 3.0, dtype=td, device=dev)
    cache = LayerCache(group=0, k=kc, v=kc)
    to = _to(dev)
    row = {s: i for i, s in enumerate(lens)}

    def run(rows, step):
        slot_map = np.concatenate([[tables[row[s], p // ps] * ps + p % ps for p in range(a, b)] for s, a, b in rows]).astype(np.int32)
        step.groups = [GroupView(ps, torch.from_numpy(tables[[row[s] for s, _, _ in rows]]).to(dev), torch.from_numpy(slot_map).to(dev))]
        x = to(np.concatenate([xs[s][a:b] for s, a, b in rows])).to(td)
        terms = [m.forward(x, step, cache, None) for m in (first, second)]
        return np.concatenate([(t.sum(0) if t.dim() == 3 else t).float().cpu().numpy() for t in terms], axis=1)
    got = _portions(dev, lens, slots, [(70, 1), (1, 2), (2, 9), (13, 1), (1, 1), (40, 40)], run)
    for s in lens:
        for g, want in ((got[s][:, :W], want1[s]), (got[s][:, W:], want2[s])):
            if dtype == "float32":
                np.testing.assert_allclose(g, want, rtol=5e-4, atol=5e-4)
            else:       # bfloat16 products: a row's difference against the row's own size (a row that the sink all but empties: against a hundredth of the rows' common size)
                e = np.sqrt(((g - want) ** 2).mean(-1)) / np.maximum(np.sqrt((want ** 2).mean(-1)), 0.01 * np.sqrt((want ** 2).mean()))
                assert e.max() < 0.05 and np.quantile(e, 0.9) < 0.02, (s, float(e.max()), int(e.argmax()))


@pytest.mark.parametrize("W,ff,limit,T", [(36, 20, 0.8, 41), (64, 72, 1.0, 9), (40, 17, 2.5, 30), (128, 256, 0.5, 70)])
def test_clamped_gated_unit_with_biases(dev, W, ff, limit, T):
    """g is clamped from above only, u on both sides; weights large enough that every bound is met by many channels."""
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import FEED_FORWARDS
    rng = np.random.default_rng(ff)
    w = _bf16_exact({"gate": rng.standard_normal((ff, W)) * 0.4, "gate.b": rng.standard_normal(ff), "up": rng.standard_normal((ff, W)) * 0.4,
                     "up.b": rng.standard_normal(ff), "down": rng.standard_normal((W, ff)) * 0.3, "down.b": rng.standard_normal(W)})
    h = rng.standard_normal((T, W))
    g, u = h @ w["gate"].T + w["gate.b"], h @ w["up"].T + w["up.b"]
    assert (g > limit).mean() > 0.02 and (g < -limit).mean() > 0.02 and (u > limit).mean() > 0.02 and (u < -limit).mean() > 0.02
    part = FEED_FORWARDS.build(PartSpec("gated_dense", {"hidden_size": W, "intermediate_size": ff, "activation": "clamped_swish", "limit": limit,
                                                        "alpha": 1.702, "bias": True}), dtype=torch.float32, device=dev)
    part.bind(lambda rel: torch.from_numpy(w[rel].astype(np.float32)))
    term = part.forward(_to(dev)(h), None)
    got = (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
    np.testing.assert_allclose(got, plain.dense(h, w, "", {"limit": limit}), rtol=3e-4, atol=3e-4)
    # the unit itself, where its pieces show: below -limit g is NOT clamped, and u + 1 is zero at u = -1
    y = plain.clamped_unit(np.array([-50.0, -3.0, 0.5, 3.0, 3.0]), np.array([9.0, -9.0, -1.0, 0.25, 9.0]), 2.0)
    sg = lambda z: 1 / (1 + np.exp(-z))
    np.testing.assert_allclose(y, [-50 * sg(-50 * 1.702) * 3, -3 * sg(-3 * 1.702) * -1, 0.0, 2 * sg(2 * 1.702) * 1.25, 2 * sg(2 * 1.702) * 3], atol=1e-12)


@pytest.mark.parametrize("E,top", [(6, 2), (8, 1), (4, 4), (3, 1), (3, 3), (64, 6), (16, 5), (40, 33), (1, 1)])
def test_router_takes_the_largest_logits_and_softmaxes_the_chosen(dev, E, top):
    import sllm_b200.ops as ops
    rng = np.random.default_rng(E + top)
    T, W = 50, 24
    h, wr = rng.standard_normal((T, W)), rng.standard_normal((E, W)) * 2.0
    chosen, weight = plain.route(h, {"router": wr}, "", {"experts": E, "top": top})
    dense, idx, wts = ops.moe_route_top_softmax(_to(dev)(h @ wr.T), top)
    want = np.zeros((T, E))
    np.put_along_axis(want, chosen, weight, axis=1)
    np.testing.assert_allclose(dense.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    assert (idx.cpu().numpy() == chosen).all()
    np.testing.assert_allclose(wts.cpu().numpy(), weight, rtol=1e-5)
    np.testing.assert_allclose(wts.sum(-1).cpu().numpy(), 1.0, rtol=1e-5)


@pytest.mark.parametrize("E,top,ff,limit", [(6, 2, 40, 1.5), (4, 4, 17, 3.0), (8, 1, 8, 0.6), (3, 2, 24, 1.0), (16, 5, 16, 2.0)])
def test_mixture_of_clamped_experts_against_plain(dev, E, top, ff, limit):
    from sllm_b200.config.plan import PartSpec
    from sllm_b200.parts import FEED_FORWARDS
    rng = np.random.default_rng(E * ff)
    W, T = 36, 41
    w = {"router": rng.standard_normal((E, W)) * 0.5}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (rng.standard_normal(s) * 0.5 for s in ((ff, W), (ff, W), (W, ff)))
    w = _bf16_exact(w)
    part = FEED_FORWARDS.build(PartSpec("gated_experts", {"hidden_size": W, "experts": E, "top": top, "expert_ff": ff, "limit": limit, "alpha": 1.702}),
                               dtype=torch.float32, device=dev)
    part.bind(lambda rel: torch.from_numpy(w[rel].astype(np.float32)))
    h = rng.standard_normal((T, W))
    term = part.forward(_to(dev)(h), None)
    got = (term.sum(0) if term.dim() == 3 else term).cpu().numpy()
    mlp = _moe(E, top, ff, limit)
    np.testing.assert_allclose(got, plain.mixture(h, w, "", mlp), rtol=3e-4, atol=3e-4)
    # a token alone gets what it gets in the batch: the experts' sum does not depend on what else the batch holds
    one = part.forward(_to(dev)(h[7:8]), None)
    np.testing.assert_allclose((one.sum(0) if one.dim() == 3 else one).cpu().numpy(), got[7:8], rtol=2e-6, atol=2e-6)


# ---- the whole model through the engine: every cutting against the plain implementation ---------------------------

def test_residual_stream_after_every_layer(tmp_path, dev):
    """The stream after each layer's last sublayer, where the next layer's norm has not yet been applied."""
    from sllm_b200.engine import build_model
    from sllm_b200.engine import Engine, StepEntry
    d = make_model(tmp_path, CONFIG_A)
    cfg, w = plain.load_model(d)
    ids = _requests(CONFIG_A["vocab"], (19,))["r0"]
    layers = []
    want = plain.forward(ids, cfg, w, layers_out=layers)
    assert len(layers) == 4
    model, _ = build_model(d, "float32", dev)
    eng = Engine(model, page_size=16, num_pages=4, max_requests=1)
    got = eng.step([StepEntry("a", ids, list(range(len(ids))))]).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=3e-4, atol=3e-4)
    # a layer less: the same weights under a configuration that stops earlier reproduce the earlier stream's logits
    for upto in (1, 3):
        short = dict(CONFIG_A, layers=CONFIG_A["layers"][:upto])
        x = plain.norm_scalar(layers[upto - 1], w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T
        np.testing.assert_allclose(plain.forward(ids, short, w), x, rtol=1e-9, atol=1e-9)


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
            if mode == "mixed" and eng.cache.groups:
                assert eng.cache.reuse_count > 0


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
    one left behind must not see that one's convolution inputs, recurrent states or latents."""
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


LONG_MEMORY = {       # every mixer can hold on to the sequence's first tokens: a head that all but never decays, gates that all but keep the state
    "architecture": "Kidolorn", "vocab": 150, "width": 128, "norm": {"eps": 1e-6}, "canon": {"taps": 3},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 32, 16, 32, 48, 0.15, 10000.0), "mlp": _dense(96, 1.0)},
        {"type": "lightning", "mixer": {"heads": 2, "dim": 64, "vdim": 32, "decay": [0.95, 0.99995]}, "mlp": None},
        {"type": "mingru", "mixer": {"width": 96}, "mlp": _dense(128, 2.0)},
        {"type": "latent_attention", "mixer": _latent(2, 64, 16, 48, 48, 0.1, 10000.0, kv_from=0), "mlp": None},
    ],
}


def _sharp(t):
    """Attention that all but picks one key, sinks that stay out of the way in one head and weigh in another, a recurrence
    whose gates all but keep the state: with these a lost key or a dropped state changes the logits by far more than the
    tolerance."""
    for n in list(t):
        if n.endswith("mix.q") and n.replace("mix.q", "mix.sink") in t:
            t[n] *= 3.0
        if n.endswith("mix.sink"):
            t[n] = t[n] * 0 + torch.linspace(-4.0, 3.0, t[n].numel())
        if n.endswith("mix.z.b"):
            t[n] = t[n] * 0.1 - 5.0
        if n.endswith("mix.o"):
            t[n] *= 2.0


def test_keys_far_back_at_page_borders_and_a_long_memory(tmp_path, dev):
    """Sharpened weights (`_sharp`): a prompt of several hundred tokens, cut at and beside page borders, then decoded
    token by token across more of them; every position wanted."""
    from sllm_b200.engine import Engine, build_model
    config, page = LONG_MEMORY, 16
    reqs = _requests(config["vocab"], (260,), seed=12)
    ids = reqs["r0"]
    for dtype, d, want, _ in models_for(tmp_path, config, dev, reqs, seed=11, edit=_sharp):
        cfg, w = plain.load_model(d)
        cut = plain.forward(ids[150:], cfg, w)              # the memory matters: without the first 150 tokens the end differs
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
        compare(tr, traces.replay_engine(tr, eng), want, dtype, f"far/{dtype}")


def test_long_decoding_from_a_short_prompt(tmp_path, dev):
    """Three tokens of prompt, then 150 tokens one at a time: the states and the cache carry everything, across many
    pages; every step's logits against the plain implementation.  The first tokens of the sequence are wanted too (the
    convolution's zeros before the start, the empty states, a softmax over one key and the sink)."""
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
            logits = plain.forward(ids, cfg, w)[-1]
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
    recipe = "tiny-kidolorn"
    if dev == "cpu":
        import yaml
        real = llm_mod.LLM
        monkeypatch.setattr(llm_mod, "LLM", lambda model_dir, **kw: real(model_dir, **dict(kw, device="cpu")))
        with open(os.path.join(cli.RECIPES_DIR, "tiny-kidolorn.yaml")) as f:
            raw = yaml.safe_load(f)
        raw["memory"] = {"kv_device_bytes": 1 << 20}
        recipe = os.path.join(str(tmp_path), "tiny-kidolorn.yaml")
        with open(recipe, "w") as f:
            yaml.safe_dump(raw, f)
    assert cli.main([recipe]) == 0
    out = capsys.readouterr().out
    assert "Kidolorn: 4 layers" in out
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
