"""Zolulix on the device against the plain implementation: every mechanism alone, whole prompts,
token-by-token decoding, portions, unequal batches, reused slots and pages, window edges, long
decoding and greedy generation through the entry point."""
import json

import numpy as np
import pytest
import torch

import plain_zolulix as pz
import sonicboom_b200 as sb
from conftest import ROOT
from sonicboom_b200 import llm, ops
from test_gpu_generate import replay
from zolulix_util import CONFIGS, latent, layer, model, recur, tokens, write_model

pytestmark = pytest.mark.gpu
# The largest root mean square of a row's difference, over the root mean square of the whole
# reference (a request's logits).  The plain implementation is float64; bfloat16 rounds to 2^-9.
# Measured on a B200 over the whole models below: float32 9.2e-6; bfloat16 2e-2 to 4e-2 for most
# requests and cuts, 8.2e-2 for the worst (activations and weights rounded to 2^-9 pass through
# two norms per sublayer; what kernel a cut's products run on moves the rounding).
TOL = {"float32": 3e-5, "bfloat16": 1.2e-1}
DTYPES = ["float32", "bfloat16"]
SEEN = {}


def rel_err(got, ref):
    ref = ref.to(torch.float64)
    ref = ref.reshape(-1, ref.shape[-1])
    d = got.to(torch.float64).cpu().reshape(ref.shape) - ref
    return float(d.pow(2).mean(-1).sqrt().max() / ref.pow(2).mean().sqrt().clamp_min(1e-30))


def model_err(got, ref, dtype):
    e = rel_err(got, ref)
    SEEN[dtype] = max(SEEN.get(dtype, 0.0), e)
    return e


def teardown_module(module):
    print("largest row errors of whole models:", {k: f"{v:.2e}" for k, v in SEEN.items()})


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"zolulix{name}")
        out[name] = (d,) + write_model(d, cfg, seed=40 + ord(name))
    return out


@pytest.fixture(scope="module")
def engines(folders):
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype)
        if key not in made:
            made[key] = sb.load_model(folders[name][0], dtype=dtype)
        return sb.Engine(made[key], max_tokens=max_tokens)
    return get


def run_cuts(engine, toks, cuts):
    """Logits at every position of one request fed in portions of the given sizes."""
    s = engine.open()
    outs, at = [], 0
    for n in cuts:
        outs.append(engine.step([(s, toks[at:at + n], list(range(n)))]).float().cpu())
        at += n
    assert at == len(toks)
    engine.close(s)
    return torch.cat(outs)


# ------------------------------------------------------------------ mechanisms alone: kernels
def test_post_norm_add_and_next_norm():
    g = torch.Generator().manual_seed(1)
    for rows, width in ((1, 8), (5, 100), (33, 1000)):
        y, x = torch.randn(rows, width, generator=g) * 3, torch.randn(rows, width, generator=g)
        w = torch.full((width,), 0.37)
        w2 = torch.randn(width, generator=g)
        ref = x.double() + pz.rms(y.double(), 1e-5) * 0.37
        out = torch.empty(rows, width, device="cuda")
        normed = torch.empty(rows, width, device="cuda", dtype=torch.bfloat16)
        ops.norm_add(y.cuda(), x.cuda(), w.cuda(), 1e-5, out, (w2.cuda(), 1e-3, normed))
        assert rel_err(out, ref) < 1e-6
        assert rel_err(normed.float(), pz.rms(ref, 1e-3) * w2.double()) < 1e-2
        plain = ops.norm_add(y.cuda(), x.cuda(), w.cuda(), 1e-5, torch.empty(rows, width, device="cuda"))
        assert torch.equal(plain, out)
        xc = x.cuda()
        assert torch.equal(ops.norm_add(y.cuda(), xc, w.cuda(), 1e-5, xc), out)       # in place


def test_depth_mix():
    g = torch.Generator().manual_seed(2)
    streams = torch.randn(7, 9, 50, generator=g)
    for n in (1, 2, 7):
        coef = torch.randn(n, generator=g)
        ref = pz.depth_sum(list(streams[:n].double()), coef.double())
        out = torch.empty(9, 50, device="cuda")
        w2 = torch.randn(50, generator=g)
        normed = torch.empty(9, 50, device="cuda")
        ops.depth_mix(streams.cuda(), n, coef.cuda(), out, (w2.cuda(), 1e-6, normed))
        assert rel_err(out, ref) < 1e-6 and rel_err(normed, pz.rms(ref, 1e-6) * w2.double()) < 1e-5
        assert torch.equal(ops.depth_mix(streams.cuda(), n, coef.bfloat16().float().cuda(), torch.empty_like(out)),
                           ops.depth_mix(streams.cuda(), n, coef.bfloat16().cuda(), torch.empty_like(out)))


def test_depth_mix_with_the_last_add():
    """The block's last residual add made inside the mix: the last stream is x + norm(y) * g."""
    g = torch.Generator().manual_seed(6)
    for rows, width, n in ((3, 40, 2), (300, 64, 5), (2, 2052, 9)):
        streams = torch.randn(n, rows, width, generator=g)
        y = torch.randn(rows, width, generator=g) * 2
        coef, w2 = torch.randn(n, generator=g), torch.randn(width, generator=g)
        gw = torch.full((width,), -0.8)
        last = streams[n - 1].double() + pz.rms(y.double(), 1e-5) * (-0.8)
        ref = pz.depth_sum(list(streams[:n - 1].double()) + [last], coef.double())
        dev = streams.cuda()
        out, normed = torch.empty(rows, width, device="cuda"), torch.empty(rows, width, device="cuda")
        ops.depth_mix(dev, n, coef.cuda(), out, (w2.cuda(), 1e-6, normed), join=(y.cuda(), dev[n - 1], gw.cuda(), 1e-5))
        assert rel_err(out, ref) < 1e-6 and rel_err(dev[n - 1], last) < 1e-6
        assert rel_err(normed, pz.rms(ref, 1e-6) * w2.double()) < 1e-5
        assert torch.equal(dev[:n - 1].cpu(), streams[:n - 1])


def test_clamped_gate_activation():
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(6, 2 * 37, generator=g) * 3
    for limit in (0.5, 1.0, 7.0):
        a, b = gu[:, :37].double().clamp(max=limit), gu[:, 37:].double().clamp(-limit, limit)
        ref = a * torch.sigmoid(1.702 * a) * (b + 1)
        out = ops.glu_clamped(gu.cuda(), limit, 1.702, torch.empty(6, 37, device="cuda"))
        assert rel_err(out, ref) < 1e-6
    assert float(gu[:, :37].max()) > 1.0 and float(gu[:, 37:].min()) < -1.0      # the clamps were in play


def test_gated_product_with_clamped_activation():
    """One product over interleaved gate and up rows whose epilogue applies the clamped activation:
    the weight-streaming kernel (few rows), the tcgen05 kernel in its decode and its many-rows
    forms, and the plain product followed by the activation kernel (float32)."""
    from sonicboom_b200.parts.feedforward import interleave_gate_up
    g = torch.Generator().manual_seed(8)
    K, ff, limit, slope = 96, 80, 0.6, 1.702
    gate, up = torch.randn(ff, K, generator=g) * 0.2, torch.randn(ff, K, generator=g) * 0.2
    for dtype in (torch.bfloat16, torch.float32):
        wg, wu = gate.to(dtype), up.to(dtype)
        w = interleave_gate_up(wg, wu).cuda()
        for rows in (3, 8, 40, 300):
            x = (torch.randn(rows, K, generator=g)).to(dtype)
            a = (x.double() @ wg.double().T).clamp(max=limit)
            b = (x.double() @ wu.double().T).clamp(-limit, limit)
            ref = a * torch.sigmoid(slope * a) * (b + 1)
            out = torch.empty(rows, ff, device="cuda", dtype=dtype)
            ops.linear(x.cuda(), w, out, ops.EPI_SWIGLU, gate=(limit, slope))
            assert rel_err(out.float(), ref) < (1e-2 if dtype == torch.bfloat16 else 1e-6), (dtype, rows)
    assert float(a.max()) == limit and float(b.min()) == -limit            # the clamps were in play


def test_head_linear():
    g = torch.Generator().manual_seed(4)
    for rows, heads, N, K in ((37, 3, 70, 19), (1, 2, 9, 100), (8, 5, 33, 40), (9, 1, 64, 16)):   # few rows: a kernel of their own
        x = torch.randn(rows, heads, K + 5, generator=g)       # a head's K values sit in a longer stretch
        w = torch.randn(heads, N, K, generator=g)
        ref = torch.einsum("rhk,hnk->rhn", x[..., 2:2 + K].double(), w.double())
        out = torch.zeros(rows, heads, N + 3, device="cuda")
        ops.head_linear(x.cuda(), 2, heads * (K + 5), K + 5, w.cuda(), out, 1, heads * (N + 3), N + 3, rows)
        assert rel_err(out[..., 1:1 + N], ref) < 1e-6
        assert float(out[..., 0].abs().max()) == 0.0 and float(out[..., N + 1:].abs().max()) == 0.0


def test_head_linear_on_tensor_cores():
    """bfloat16 weights and outputs at many rows: float32 and bfloat16 inputs, rows and outputs that
    end inside a tile, a head's values inside a longer stretch."""
    g = torch.Generator().manual_seed(5)
    for rows, heads, N, K, in_dtype in ((70, 3, 40, 32, torch.float32), (200, 2, 130, 48, torch.bfloat16),
                                        (9, 5, 64, 16, torch.float32)):
        x = torch.randn(rows, heads, K + 6, generator=g).to(in_dtype)
        w = torch.randn(heads, N, K, generator=g).bfloat16()
        ref = torch.einsum("rhk,hnk->rhn", x[..., 2:2 + K].bfloat16().double(), w.double())
        out = torch.zeros(rows, heads, N + 4, device="cuda", dtype=torch.bfloat16)
        ops.head_linear(x.cuda(), 2, heads * (K + 6), K + 6, w.cuda(), out, 2, heads * (N + 4), N + 4, rows)
        assert rel_err(out[..., 2:2 + N].float(), ref) < 1e-2
        assert float(out[..., :2].abs().max()) == 0.0 and float(out[..., N + 2:].abs().max()) == 0.0


# ------------------------------------------------------------------ mechanisms alone: one-layer models
ONE_LAYER = {
    "latent": model(64, 32, [layer("latent_attention", latent(2, 8, 8, 12, 24, window=11, dims=6))]),
    "latent_wide": model(64, 32, [layer("latent_attention", latent(3, 16, 16, 8, 48, window=200))]),
    # a latent width of 128 (the tensor-memory attention kernels) and of 144; twenty heads on one
    # key/value head (single tokens then run the kernel for many rows)
    "latent_128": model(64, 32, [layer("latent_attention", latent(4, 32, 32, 32, 96, window=50))]),
    "latent_20_heads": model(64, 32, [layer("latent_attention", latent(20, 8, 16, 8, 128, window=70))]),
    # widths and inner sizes that are no multiple of 8: the plain products in both dtypes
    "odd_sizes": model(61, 44, [layer("latent_attention", latent(3, 12, 4, 7, 20, window=30), ff=20, limit=0.9),
                                layer("mlstm", recur(3, 10, 7), ff=36, limit=1.1)]),
    "mlstm": model(64, 32, [layer("mlstm", recur(2, 16, 9, cap=6.0))]),
    # key sizes served by 16 x 16 and by 32 lanes a column
    "mlstm_dim_200": model(64, 32, [layer("mlstm", recur(1, 200, 17))]),
    "mlstm_dim_300": model(64, 32, [layer("mlstm", recur(2, 300, 33))]),
    "mlstm_any_dim": model(64, 32, [layer("mlstm", recur(1, 20, 130, cap=20.0))]),
    "ff": model(64, 32, [layer("mlstm", recur(1, 16, 24)), layer("mlstm", recur(1, 16, 24), ff=24, limit=0.3)]),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_in_a_model_of_its_own(tmp_path, name, dtype):
    cfg, tensors = write_model(tmp_path / name, ONE_LAYER[name], seed=7)
    toks = tokens(cfg, 90, 3)
    streams = []
    ref = pz.forward(cfg, tensors, toks, streams)
    engine = sb.Engine(sb.load_model(tmp_path / name, dtype=dtype), max_tokens=256)
    assert model_err(run_cuts(engine, toks, [90]), ref, dtype) < TOL[dtype]
    assert model_err(run_cuts(engine, toks, [50] + [1] * 40), ref, dtype) < TOL[dtype]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decoding_and_portions(folders, engines, name, dtype):
    _, cfg, tensors = folders[name]
    toks = tokens(cfg, 171, 5)
    ref = pz.forward(cfg, tensors, toks)
    engine = engines(name, dtype)
    whole = run_cuts(engine, toks, [171])
    assert model_err(whole, ref, dtype) < TOL[dtype]
    # the first tokens of a sequence one by one, then the rest; most of it at once, then one by one
    # over two page borders (64, 128) and every window's edge; portions down to two tokens
    for cuts in ([1, 1, 1, 168], [40] + [1] * 131, [2, 3, 62, 2, 59, 7, 17, 19], [64, 64, 43], [170, 1]):
        got = run_cuts(engine, toks, cuts)
        assert model_err(got, ref, dtype) < TOL[dtype], cuts
        if dtype == "float32":
            assert rel_err(got, whole) < 1e-5, cuts       # rounding: few rows run other kernels
    engine.cache.check()
    assert engine.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_equals_each_alone_and_slots_are_reused(folders, engines, name, dtype):
    from gpu_util import batch_unequal
    _, cfg, tensors = folders[name]
    reqs = [tokens(cfg, n, 10 + n) for n in (1, 70, 131, 23)]
    refs = [pz.forward(cfg, tensors, r) for r in reqs]
    engine = engines(name, dtype, max_tokens=512)
    # twice in the same engine: the second pass reuses the slots, pages and state rows of the first
    for _ in range(2):
        outs = batch_unequal(engine, reqs, [1, 40, 100, 23])
        for o, r in zip(outs, refs):
            assert model_err(o, r, dtype) < TOL[dtype]
        engine.cache.check()
    alone = [run_cuts(engine, r, [k] + [1] * (len(r) - k)) for r, k in zip(reqs, [1, 40, 100, 23])]
    if dtype == "float32":
        for o, a in zip(outs, alone):
            assert rel_err(o, a) < 1e-5
    # a sequence that ends early gives its slot to a new one while the others go on
    a, b = engine.open(), engine.open()
    engine.step([(a, reqs[1][:30], []), (b, reqs[2][:50], [])])
    engine.close(a)
    c = engine.open()
    assert c == a
    lg = engine.step([(b, reqs[2][50:60], list(range(10))), (c, reqs[3], list(range(23)))]).float().cpu()
    assert rel_err(lg[:10], refs[2][50:60]) < TOL[dtype] and rel_err(lg[10:], refs[3]) < TOL[dtype]
    engine.close(b), engine.close(c)


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_show(tmp_path, dtype):
    """Queries and keys scaled up so that single keys stand out: were a window one key too long
    or too short, or a far key lost, logits would move by far more than the tolerance."""
    base = model(80, 48, [
        layer("latent_attention", latent(2, 16, 16, 16, 32, window=13, scale=1.0)),
        layer("latent_attention", latent(2, 16, 16, 16, 32, window=70, scale=1.0, kv_from=0)),
    ])

    def sharpen(t):
        for i in (0, 1):
            t[f"l{i}.mix.q"] *= 4.0
    cfg, tensors = write_model(tmp_path / "w", base, seed=9, edit=sharpen)
    toks = tokens(cfg, 160, 21)
    ref = pz.forward(cfg, tensors, toks)
    for which, delta in ((0, 1), (0, -1), (1, 1), (1, -1)):
        other = json.loads(json.dumps(cfg))
        other["layers"][which]["mixer"]["mask"]["size"] += delta
        assert rel_err(pz.forward(other, tensors, toks)[80:], ref[80:]) > 4 * TOL[dtype], (which, delta)
    engine = sb.Engine(sb.load_model(tmp_path / "w", dtype=dtype), max_tokens=512)
    for cuts in ([160], [60] + [1] * 100, [12, 2, 50, 96], [13] + [1] * 147):
        assert rel_err(run_cuts(engine, toks, cuts), ref) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_keeps_the_state(folders, engines, dtype):
    """Six hundred tokens one by one: the window passes over many pages (which are given back),
    the recurrence's state is carried all the way."""
    _, cfg, tensors = folders["Q"]
    toks = tokens(cfg, 600, 77)
    ref = pz.forward(cfg, tensors, toks)
    engine = engines("Q", dtype, max_tokens=256)        # far fewer pages than 600 tokens would hold
    s = engine.open()
    engine.step([(s, toks[:5], [])])
    rows = []
    for i in range(5, 600):
        lg = engine.step([(s, [toks[i]], [0] if i % 7 == 0 or i > 590 else [])])
        if lg is not None:
            rows.append((i, lg.float().cpu()[0]))
    engine.close(s)
    got = torch.stack([r for _, r in rows])
    assert rel_err(got, ref[[i for i, _ in rows]]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """`llm.generate_batch`: the scheduler's batches, the captured decode step with the
    recurrence's state in it, and slots given to the next batch."""
    d, cfg, tensors = folders[name]
    m = llm.model_load(d, dtype=dtype)
    assert m.arch == "Zolulix" and m.vocab_size == cfg["vocab"]
    prompts = [tokens(cfg, n, 30 + n) for n in (3, 66, 20, 1)]
    n_new = 12
    outs = llm.generate_batch(m, prompts, max_tokens=n_new)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for i, t in enumerate(o):
            logits = pz.forward(cfg, tensors, seq)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                top2 = torch.topk(logits, 2).values
                margin = float(top2[0] - top2[1]) / float(logits.abs().max())
                assert dtype == "bfloat16" and margin < 2 * TOL[dtype], (i, o, margin)
                break
            seq.append(t)
    alone = [llm.generate_batch(m, [p], max_tokens=n_new)[0] for p in prompts]
    small = llm.generate_batch(m, prompts, max_tokens=n_new, max_cache_tokens=192)     # more than one batch
    if dtype == "float32":
        assert alone == outs and small == outs
    s = llm.session_new(m, 128)
    assert llm.generate_tokens(s, prompts[2], n_new) == alone[2]
    s.free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_program(folders, tmp_path, dtype):
    d, cfg, tensors = folders["P"]
    a, b = tokens(cfg, 75, 1), tokens(cfg, 30, 2)
    ra, rb = pz.forward(cfg, tensors, a).numpy(), pz.forward(cfg, tensors, b).numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]},
                                     {"id": "b", "tokens": b[:29], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:71], "want": [0]},
                                     {"id": "b", "tokens": b[29:], "want": [0]}], "end": ["b"]}]
    steps += [{"step": i - 69, "entries": [{"id": "a", "tokens": [a[i]], "want": [0] if i % 2 else []}],
               "end": ["a"] if i == 74 else []} for i in range(71, 75)]
    got = replay(d, dtype, steps, tmp_path / "out", 256)
    V = cfg["vocab"]
    want = {0: ra[[0, 69]], 1: np.stack([ra[70], rb[29]]), 2: ra[71:72], 4: ra[73:74]}
    assert set(got) == set(want)
    for k, ref in want.items():
        assert np.abs(got[k].reshape(-1, V) - ref).max() / np.abs(ra).max() < TOL[dtype], k
