"""Mefupel on the device against the plain implementation: every mechanism alone (kernels, then
one-layer models), whole prompts, token-by-token decoding, portions, unequal batches, reused
slots, pages and state rows, window edges, far keys, long decoding, greedy generation through
the entry point and the trace replay program."""
import json

import numpy as np
import pytest
import torch

import plain_mefupel as pf
import sonicboom_b200 as sb
from sonicboom_b200 import llm, ops
from sonicboom_b200.cache.kv import Cache, KVNeed
from sonicboom_b200.engine.step import StepEntry, StepPlan
from sonicboom_b200.parts.rotary import frequency_table
from test_gpu_generate import replay
from mefupel_util import CONFIGS, attention, gla, layer, model, retention, tokens, write_model

pytestmark = pytest.mark.gpu
# The largest root mean square of a row's difference, over the root mean square of the whole
# reference (a request's logits).  The plain implementation is float64; bfloat16 rounds to 2^-9.
# Measured on a B200 over the whole models below: float32 9.3e-6; bfloat16 1e-2 to 3e-2 for most
# requests and cuts, 5.9e-2 for the worst (a row where a recurrence's sum nearly cancels before its
# head is divided by its root mean square carries the rounding of its inputs much enlarged).
TOL = {"float32": 3e-5, "bfloat16": 8e-2}
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
SEEN = {}
F = torch.float64


def rel_err(got, ref):
    ref = ref.to(F)
    ref = ref.reshape(-1, ref.shape[-1])
    d = got.to(F).cpu().reshape(ref.shape) - ref
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
        d = tmp_path_factory.mktemp(f"mefupel{name}")
        out[name] = (d,) + write_model(d, cfg, seed=60 + ord(name))
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
def test_a_vector_joins_the_stream():
    g = torch.Generator().manual_seed(1)
    for rows, width in ((1, 8), (5, 100), (40, 1000)):
        x, e = torch.randn(rows, width, generator=g), torch.randn(rows, width, generator=g)
        vec, w2 = torch.randn(width, generator=g).bfloat16(), torch.randn(width, generator=g)
        ref = x.double() + e.double() + vec.double()
        out = torch.empty(rows, width, device="cuda")
        normed = torch.empty(rows, width, device="cuda")
        ops.stream_add(x.cuda(), e.cuda(), vec.cuda(), out, (w2.cuda(), 1e-3, normed))
        assert rel_err(out, ref) < 1e-6 and rel_err(normed, pf.rms(ref, 1e-3) * w2.double()) < 1e-5
        xc = x.cuda()
        assert torch.equal(ops.stream_add(xc, e.cuda(), vec.cuda(), xc), out)           # in place
        assert rel_err(ops.stream_add(x.cuda(), None, vec.cuda(), torch.empty_like(out)), x.double() + vec.double()) < 1e-6
        assert torch.equal(ops.stream_add(x.cuda(), None, None, torch.empty_like(out)).cpu(), x)


def test_polynorm_activation():
    g = torch.Generator().manual_seed(2)
    coef = torch.tensor([0.7, -0.4, 0.2, 0.1])
    for rows, ff in ((3, 7), (9, 300), (2, 5000), (600, 64)):
        z = torch.randn(rows, ff, generator=g) * 2
        zz = z.double()
        ref = 0.7 * pf.rms(zz, 1e-5) - 0.4 * pf.rms(zz ** 2, 1e-5) + 0.2 * pf.rms(zz ** 3, 1e-5) + 0.1
        out = ops.polynorm(z.cuda(), coef.cuda(), 1e-5, torch.empty(rows, ff, device="cuda"))
        assert rel_err(out, ref) < 2e-6
        out16 = ops.polynorm(z.cuda(), coef.bfloat16().cuda(), 1e-5, torch.empty(rows, ff, device="cuda", dtype=torch.bfloat16))
        c16 = coef.bfloat16().double()
        ref16 = c16[0] * pf.rms(zz, 1e-5) + c16[1] * pf.rms(zz ** 2, 1e-5) + c16[2] * pf.rms(zz ** 3, 1e-5) + c16[3]
        assert rel_err(out16.float(), ref16) < 1e-2


def attend(dtype, seqs, hq, hkv, dim, vdim, window, scale, rot, layout, base, rotate_values, qk_norm, keys_as_values,
           sink, kernel="auto", eps=1e-5, cache=None, slots=None):
    """Projection rows of several sequences (float32 [n, q | k | v]) through `attn_prep`, the
    attention kernels and `attn_unrotate`; returns [rows, hq * vdim]."""
    hd = (max(dim, vdim) + 15) // 16 * 16
    if cache is None:
        cache = Cache([KVNeed(hkv, hd, window)], [None], 4096, DT[dtype], "cuda")
        slots = [cache.open() for _ in seqs]
    for s, x in zip(slots, seqs):
        cache.reserve(s, cache.length(s) + x.shape[0])
    plan = StepPlan(cache, [StepEntry(s, [0] * x.shape[0], []) for s, x in zip(slots, seqs)], "cuda")
    proj = torch.cat(seqs).cuda()
    g, storage = plan.groups[0], cache.groups[0].entry_storage(0)
    q = torch.empty(proj.shape[0], hq, hd, dtype=DT[dtype], device="cuda")
    inter = layout == "interleaved"
    ops.attn_prep(proj, 0, hq * dim, -1 if keys_as_values else (hq + hkv) * dim, hq, hkv, dim, vdim, hd, rot, inter,
                  frequency_table(base, rot, "cuda") if rot else None,
                  frequency_table(base, vdim, "cuda") if rotate_values else None,
                  qk_norm[0].cuda() if qk_norm else None, qk_norm[1].cuda() if qk_norm else None, eps,
                  plan.row_seq, plan.row_pos, g.page_off, g.page_ids, g.page_size, storage, q)
    out = torch.empty(proj.shape[0], hq * hd, dtype=DT[dtype], device="cuda")
    ops.attention(q, out, plan, 0, storage, hq, hkv, hd, window, scale, kernel=kernel,
                  sink=sink.cuda() if sink is not None else None)
    if rotate_values or hd != vdim:
        out = ops.attn_unrotate(out, torch.empty(proj.shape[0], hq * vdim, dtype=DT[dtype], device="cuda"), hq, hd,
                                vdim, inter, frequency_table(base, vdim, "cuda") if rotate_values else None, plan.row_pos)
    for s, x in zip(slots, seqs):
        cache.advance(s, cache.length(s) + x.shape[0])
    return out.float().cpu(), cache, slots


def attend_ref(x, hq, hkv, dim, vdim, window, scale, rot, layout, base, rotate_values, qk_norm, keys_as_values, sink,
               eps=1e-5):
    """The same on one whole sequence with the plain implementation's functions."""
    x = x.double()
    T = x.shape[0]
    pos = torch.arange(T)
    q_raw, k_raw = x[:, :hq * dim], x[:, hq * dim:(hq + hkv) * dim]
    v = (k_raw if keys_as_values else x[:, (hq + hkv) * dim:]).reshape(T, hkv, vdim)
    if qk_norm:
        q_raw, k_raw = pf.rms(q_raw, eps) * qk_norm[0].double(), pf.rms(k_raw, eps) * qk_norm[1].double()
    q = pf.rotate(q_raw.reshape(T, hq, dim), pos, base, rot, layout)
    k = pf.rotate(k_raw.reshape(T, hkv, dim), pos, base, rot, layout)
    if rotate_values:
        v = pf.rotate(v, pos, base, vdim, layout)
    o = pf.windowed_softmax_attention(q, k, v, scale, window, sink=sink.double() if sink is not None else None)
    if rotate_values:
        o = pf.rotate(o, pos, base, vdim, layout, sign=-1.0)
    return o.reshape(T, hq * vdim)


ATTENTION_CASES = {
    # values wider than keys, rotated; a rotated prefix; interleaved pairs
    "rotated_values": dict(hq=4, hkv=2, dim=16, vdim=24, window=9, scale=0.4, rot=8, layout="interleaved",
                           base=100.0, rotate_values=True, qk_norm=False, keys_as_values=False, sink=False),
    # values narrower than keys, head size 40 padded to 48, no rotation of keys at all
    "narrow_values": dict(hq=3, hkv=3, dim=40, vdim=10, window=70, scale=0.2, rot=0, layout="halves", base=10000.0,
                          rotate_values=True, qk_norm=False, keys_as_values=False, sink=False),
    # keys as values, whole-projection norms, a sink, halves; head sizes of the mma.sync and of the tensor-memory kernels
    "sink_32": dict(hq=4, hkv=1, dim=32, vdim=32, window=20, scale=0.3, rot=16, layout="halves", base=10000.0,
                    rotate_values=False, qk_norm=True, keys_as_values=True, sink=True),
    "sink_64": dict(hq=4, hkv=2, dim=64, vdim=64, window=130, scale=0.2, rot=64, layout="halves", base=2e6,
                    rotate_values=False, qk_norm=True, keys_as_values=True, sink=True),
    "sink_128": dict(hq=6, hkv=2, dim=128, vdim=128, window=100, scale=0.15, rot=64, layout="halves", base=1e4,
                     rotate_values=False, qk_norm=True, keys_as_values=True, sink=True),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kernel", ["auto", "plain", "mma", "tma"])
@pytest.mark.parametrize("case", list(ATTENTION_CASES))
def test_attention_rows_in_and_out(case, kernel, dtype):
    """A prompt of 300 tokens, then 40 tokens one by one with a second, shorter sequence beside it,
    on every attention kernel: the plain one, mma.sync, tensor memory (prefill) and TMA (decode)."""
    if dtype == "float32" and kernel != "auto":
        pytest.skip("float32 runs the plain kernel whatever is asked for")
    c = dict(ATTENTION_CASES[case])
    g = torch.Generator().manual_seed(len(case))
    hq, hkv, dim, vdim = c["hq"], c["hkv"], c["dim"], c["vdim"]
    width = (hq + hkv) * dim + (0 if c["keys_as_values"] else hkv * vdim)
    xa, xb = torch.randn(340, width, generator=g), torch.randn(90, width, generator=g)
    c["qk_norm"] = (1 + 0.3 * torch.randn(hq * dim, generator=g), 1 + 0.3 * torch.randn(hkv * dim, generator=g)) \
        if c["qk_norm"] else None
    c["sink"] = torch.randn(hq, generator=g) * 2 + 1 if c["sink"] else None
    ref_a, ref_b = attend_ref(xa, **c), attend_ref(xb, **c)
    got_a, cache, slots = attend(dtype, [xa[:300], xb[:50]], kernel=kernel, **c)
    rows_a, rows_b = [got_a[:300]], [got_a[300:]]
    for i in range(40):
        o, _, _ = attend(dtype, [xa[300 + i:301 + i], xb[50 + i:51 + i]], kernel=kernel, cache=cache, slots=slots, **c)
        rows_a.append(o[:1]), rows_b.append(o[1:])
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert rel_err(torch.cat(rows_a), ref_a) < tol and rel_err(torch.cat(rows_b), ref_b) < tol


def test_a_sink_that_outweighs_every_key_shows():
    """With a large sink the result shrinks towards zero; were it left out, the rows would be the
    plain softmax's."""
    c = dict(ATTENTION_CASES["sink_64"])
    g = torch.Generator().manual_seed(5)
    x = torch.randn(200, (c["hq"] + c["hkv"]) * 64, generator=g)
    c["qk_norm"] = None
    none = dict(c, sink=None)
    c["sink"] = torch.full((c["hq"],), 6.0)
    ref, without = attend_ref(x, **c), attend_ref(x, **none)
    assert rel_err(without, ref) > 1.0
    for kernel in ("auto", "mma", "plain"):
        got, _, _ = attend("bfloat16", [x], kernel=kernel, **c)
        assert rel_err(got, ref) < 2e-2, kernel


def scan(seqs_proj, H, d, dv, decay, head_decay, state, slots, q_scale=1.0, k_scale=1.0, rot=0, layout="halves",
         base=10000.0, pos0=None, z=None, tau=1.0, norm_w=None, eps=1e-5, out_dtype=torch.float32):
    """Projection rows [n, q | k | v | g] of several sequences through prep, scan and out."""
    class P:
        pass
    plan = P()
    lens = [x.shape[0] for x in seqs_proj]
    plan.n_seqs = len(lens)
    plan.seq_row0 = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    plan.seq_slot = torch.tensor(slots, dtype=torch.int32, device="cuda")
    pos0 = pos0 or [0] * len(lens)
    row_pos = torch.tensor(np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, lens)]), dtype=torch.int32, device="cuda")
    proj = torch.cat(seqs_proj).cuda().contiguous()
    zz = torch.cat(z).cuda().contiguous() if z is not None else None
    ops.linrec_prep(proj, 0, H * d, H, d, q_scale, k_scale, rot, layout == "interleaved",
                    frequency_table(base, rot, "cuda") if rot else None, row_pos, zz, 1.0 / tau)
    o = torch.empty(proj.shape[0], H, dv, device="cuda")
    ops.linrec_scan(proj, 0, H * d, 2 * H * d, plan, H, d, dv, zz,
                    torch.tensor(head_decay, dtype=torch.float32, device="cuda") if head_decay is not None else None, state, o)
    out = torch.empty(proj.shape[0], H * dv, device="cuda", dtype=out_dtype)
    ops.linrec_out(o, proj, 2 * H * d + H * dv, H, dv, norm_w.cuda() if norm_w is not None else None, eps, out)
    return out.float().cpu()


@pytest.mark.parametrize("H,d,dv", [(2, 16, 12), (1, 24, 40), (3, 40, 33), (2, 64, 64), (1, 128, 9), (1, 200, 17), (5, 5, 3), (1, 300, 10)])
def test_linear_recurrence_kernels(H, d, dv):
    """Both kinds of decay; prompts against token by token; two sequences side by side in slots
    that are not in order; key sizes on every register variant and between them."""
    g = torch.Generator().manual_seed(H * 1000 + d)
    T = 70
    width = 2 * H * d + 2 * H * dv
    xs = [torch.randn(T, width, generator=g) * 0.5, torch.randn(T - 20, width, generator=g) * 0.5]
    zs = [torch.randn(x.shape[0], H * d, generator=g) * 2 for x in xs]
    norm_w = 1 + 0.2 * torch.randn(dv, generator=g)
    rot = d // 2 * 2 if d % 4 == 0 else 0
    for kind in ("channel", "head"):
        hd = [0.5 + 0.49 * (i + 1) / H for i in range(H)] if kind == "head" else None
        refs = []
        for x, z in zip(xs, zs):
            n = x.shape[0]
            pos = torch.arange(n)
            xd = x.double()
            q = pf.rotate(xd[:, :H * d].reshape(n, H, d), pos, 1000.0, rot, "halves") * 0.7
            k = pf.rotate(xd[:, H * d:2 * H * d].reshape(n, H, d), pos, 1000.0, rot, "halves") * 1.3
            v = xd[:, 2 * H * d:2 * H * d + H * dv].reshape(n, H, dv)
            gate = xd[:, 2 * H * d + H * dv:]
            a = torch.exp(torch.nn.functional.logsigmoid(z.double()) / 4.0).reshape(n, H, d) if kind == "channel" else \
                torch.tensor(hd, dtype=F)[None, :, None].expand(n, H, d)
            o = pf.rms(pf.linear_recurrence(q, k, v, a), 1e-5)
            if kind == "channel":
                o = o * norm_w.double()
            refs.append(o.reshape(n, H * dv) * gate * torch.sigmoid(gate))
        kw = dict(q_scale=0.7, k_scale=1.3, rot=rot, base=1000.0, tau=4.0, norm_w=norm_w if kind == "channel" else None)
        state = torch.zeros(6, H, dv, d, device="cuda")
        whole = scan(xs, H, d, dv, None, hd, state, [4, 1], z=zs if kind == "channel" else None, **kw)
        assert rel_err(whole[:T], refs[0]) < 1e-5 and rel_err(whole[T:], refs[1]) < 1e-5
        assert float(state[[0, 2, 3, 5]].abs().max()) == 0.0
        # one or two columns of the state per thread: the same bits
        for cpt in (1, 2):
            ops.force_linrec_columns(cpt)
            again = torch.zeros(6, H, dv, d, device="cuda")
            try:
                assert torch.equal(scan(xs, H, d, dv, None, hd, again, [4, 1], z=zs if kind == "channel" else None, **kw), whole)
            finally:
                ops.force_linrec_columns(0)
            assert torch.equal(again, state)
        # the same in portions of 30, 2, 1, 1, ... tokens from a fresh state, the other slot order
        state2 = torch.zeros(6, H, dv, d, device="cuda")
        outs, at = [[], []], [0, 0]
        for n in [30, 2] + [1] * 38:
            live = [i for i in (0, 1) if at[i] < xs[i].shape[0]]
            take = [min(n, xs[i].shape[0] - at[i]) for i in live]
            o = scan([xs[i][at[i]:at[i] + t] for i, t in zip(live, take)], H, d, dv, None, hd, state2,
                     [[2, 5][i] for i in live], pos0=[at[i] for i in live],
                     z=[zs[i][at[i]:at[i] + t] for i, t in zip(live, take)] if kind == "channel" else None, **kw)
            r = 0
            for i, t in zip(live, take):
                outs[i].append(o[r:r + t])
                r += t
                at[i] += t
        assert torch.equal(torch.cat(outs[0]), whole[:T]) and torch.equal(torch.cat(outs[1]), whole[T:])
        assert torch.equal(state2[2], state[4]) and torch.equal(state2[5], state[1])


def test_decay_map_in_the_prep_kernel():
    """The second half of the low-rank decay map, worked out where the decays are made."""
    g = torch.Generator().manual_seed(12)
    for rows, H, d, rank, dt in ((5, 2, 16, 4, torch.float32), (70, 3, 40, 24, torch.bfloat16), (9, 1, 8, 1, torch.bfloat16)):
        extra = 11
        proj = torch.randn(rows, 2 * H * d + extra + rank, generator=g)
        a2, b = (torch.randn(H * d, rank, generator=g) * 0.5).to(dt), torch.randn(H * d, generator=g).to(dt)
        zl = b.double() + proj[:, 2 * H * d + extra:].double() @ a2.double().T
        ref = torch.exp(torch.nn.functional.logsigmoid(zl) / 3.0)
        dev = proj.cuda()
        z = torch.empty(rows, H * d, device="cuda")
        pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
        ops.linrec_prep(dev, 0, H * d, H, d, 2.0, 0.5, 0, False, None, pos, z, 1.0 / 3.0,
                        low_rank=(a2.cuda(), b.cuda(), 2 * H * d + extra))
        assert rel_err(z, ref) < 1e-6
        assert rel_err(dev[:, :H * d], proj[:, :H * d].double() * 2.0) < 1e-7
        assert rel_err(dev[:, H * d:2 * H * d], proj[:, H * d:2 * H * d].double() * 0.5) < 1e-7
        assert torch.equal(dev[:, 2 * H * d:].cpu(), proj[:, 2 * H * d:])


# ------------------------------------------------------------------ mechanisms alone: one-layer models
ONE_LAYER = {
    "attention": model(64, 32, [layer("attention", attention(2, 1, 16, 16, window=11, dims=6))]),
    "attention_wide_values": model(64, 32, [layer("attention", attention(3, 3, 8, 40, window=200, base=50.0))]),
    "attention_128": model(64, 32, [layer("attention", attention(2, 2, 128, 128, window=50, dims=32))]),
    "gla": model(64, 32, [layer("gla", gla(2, 16, 9, tau=3.0, rank=5))]),
    "gla_long_memory": model(64, 32, [layer("gla", gla(1, 48, 20, tau=64.0, rank=8))]),
    "side_by_side": model(64, 32, [layer("parallel", {"left": attention(2, 1, 16, 16, window=13, dims=8),
                                                     "right": retention(2, 8, 12, [0.8, 0.99], dims=4)})]),
    "side_by_side_128": model(64, 32, [layer("parallel", {"left": attention(4, 2, 128, 128, window=40, dims=64),
                                                         "right": retention(1, 64, 64, [0.995])})]),
    "ff": model(64, 32, [layer("gla", gla(1, 16, 8), ff=24), layer("gla", gla(1, 16, 8))]),
    # widths and inner sizes that are no multiple of 8: the plain products in both dtypes
    "odd_sizes": model(61, 44, [layer("attention", attention(3, 1, 12, 6, window=30, dims=4), ff=20),
                                layer("parallel", {"left": attention(2, 2, 10, 10, window=7, dims=10),
                                                   "right": retention(3, 10, 7, [0.9, 0.5, 0.99], dims=6)}, ff=36)]),
    "loop_of_one": model(64, 32, [layer("gla", gla(2, 8, 8), ff=16)], loop=(0, 1, 4)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_in_a_model_of_its_own(tmp_path, name, dtype):
    cfg, tensors = write_model(tmp_path / name, ONE_LAYER[name], seed=7)
    toks = tokens(cfg, 90, 3)
    ref = pf.forward(cfg, tensors, toks)
    engine = sb.Engine(sb.load_model(tmp_path / name, dtype=dtype), max_tokens=256)
    assert model_err(run_cuts(engine, toks, [90]), ref, dtype) < TOL[dtype]
    assert model_err(run_cuts(engine, toks, [50] + [1] * 40), ref, dtype) < TOL[dtype]


def test_the_stream_after_every_layer(folders, engines):
    """float32: the residual stream after every schedule entry against the plain implementation's."""
    _, cfg, tensors = folders["A"]
    toks = tokens(cfg, 40, 8)
    streams = []
    pf.forward(cfg, tensors, toks, streams)
    engine = engines("A", "float32")
    seen = []
    blocks = engine.model.blocks
    originals = [b.forward for b in blocks]
    for b, orig in zip(blocks, originals):
        b.forward = lambda x, ctx, orig=orig: (lambda y: (seen.append(y.clone()), y)[1])(orig(x, ctx))
    try:
        run_cuts(engine, toks, [40])
    finally:
        for b in blocks:
            del b.forward
    assert len(seen) == len(streams) == 8
    for i, (got, ref) in enumerate(zip(seen, streams)):
        assert rel_err(got, ref) < 1e-5, i


def test_the_rank_of_the_decay_map_may_come_from_the_file(tmp_path):
    cfg, tensors = write_model(tmp_path / "m", ONE_LAYER["gla"], seed=3, drop_rank=True)
    assert "decay_rank" not in cfg["layers"][0]["mixer"]
    toks = tokens(cfg, 30, 1)
    engine = sb.Engine(sb.load_model(tmp_path / "m", dtype="float32"), max_tokens=128)
    assert rel_err(run_cuts(engine, toks, [30]), pf.forward(cfg, tensors, toks)) < TOL["float32"]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decoding_and_portions(folders, engines, name, dtype):
    _, cfg, tensors = folders[name]
    toks = tokens(cfg, 171, 5)
    ref = pf.forward(cfg, tensors, toks)
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
    refs = [pf.forward(cfg, tensors, r) for r in reqs]
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
def test_window_edges_and_sinks_show(tmp_path, dtype):
    """Queries scaled up so that single keys stand out: were a window one key too long or too
    short, a far key lost or a sink left out, logits would move by far more than the tolerance."""
    base = model(80, 48, [
        layer("attention", attention(2, 1, 16, 16, window=13, scale=1.0)),
        layer("parallel", {"left": attention(2, 2, 32, 32, window=70, dims=16, scale=1.0),
                           "right": retention(1, 16, 16, [0.99])}),
    ])

    def sharpen(t):
        t["l0.mix.q"] *= 2.5
        t["l1.mix.left.q.norm"] *= 2.0
    cfg, tensors = write_model(tmp_path / "w", base, seed=9, edit=sharpen)
    toks = tokens(cfg, 160, 21)
    ref = pf.forward(cfg, tensors, toks)
    # sharpened scores carry bfloat16's rounding of queries and keys further (0.084 measured)
    tol = TOL[dtype] * (1.5 if dtype == "bfloat16" else 1.0)
    for which, delta in ((0, 1), (0, -1), (1, 1), (1, -1)):
        other = json.loads(json.dumps(cfg))
        m = other["layers"][which]["mixer"]
        (m if which == 0 else m["left"])["mask"]["size"] += delta
        assert rel_err(pf.forward(other, tensors, toks)[80:], ref[80:]) > 4 * tol, (which, delta)
    no_sink = dict(tensors)
    no_sink["l1.mix.left.sink"] = torch.full_like(tensors["l1.mix.left.sink"], -60.0)
    assert rel_err(pf.forward(cfg, no_sink, toks), ref) > 2.5 * tol
    engine = sb.Engine(sb.load_model(tmp_path / "w", dtype=dtype), max_tokens=512)
    for cuts in ([160], [60] + [1] * 100, [12, 2, 50, 96], [13] + [1] * 147):
        assert rel_err(run_cuts(engine, toks, cuts), ref) < tol, cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_stays_in_the_state(tmp_path, dtype):
    """Decays close to one: four hundred tokens later the logits still depend on the fourth token
    (by 2e-2 of their size: a thousand times the float32 tolerance, which is where a lost or
    reset state would show), through prompts and through single tokens."""
    base = model(70, 32, [layer("parallel", {"left": attention(1, 1, 16, 16, window=4),
                                             "right": retention(2, 16, 16, [0.9995, 0.999], dims=0)}),
                          layer("gla", gla(1, 16, 16, tau=200.0, rank=4))])

    def loud(t):
        t["l0.mix.right.out"] *= 4.0
        t["l1.mix.a2.b"] += 4.0
    cfg, tensors = write_model(tmp_path / "far", base, seed=11, edit=loud)
    toks = tokens(cfg, 420, 2)
    other = list(toks)
    other[3] = (toks[3] + 1) % cfg["vocab"]
    ref = pf.forward(cfg, tensors, toks)
    assert rel_err(pf.forward(cfg, tensors, other)[400:], ref[400:]) > 500 * TOL["float32"]
    engine = sb.Engine(sb.load_model(tmp_path / "far", dtype=dtype), max_tokens=512)
    for cuts in ([420], [380] + [1] * 40, [5, 200, 215]):
        assert rel_err(run_cuts(engine, toks, cuts)[400:], ref[400:]) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_keeps_the_state(folders, engines, dtype):
    """Six hundred tokens one by one: the windows pass over many pages (which are given back),
    the recurrences' states are carried all the way."""
    _, cfg, tensors = folders["A"]
    toks = tokens(cfg, 600, 77)
    ref = pf.forward(cfg, tensors, toks)
    engine = engines("A", dtype, max_tokens=320)        # far fewer pages than 600 tokens would hold
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
    recurrences' states in it, and slots given to the next batch."""
    d, cfg, tensors = folders[name]
    m = llm.model_load(d, dtype=dtype)
    assert m.arch == "Mefupel" and m.vocab_size == cfg["vocab"]
    prompts = [tokens(cfg, n, 30 + n) for n in (3, 66, 20, 1)]
    n_new = 12
    outs = llm.generate_batch(m, prompts, max_tokens=n_new)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for i, t in enumerate(o):
            logits = pf.forward(cfg, tensors, seq)[-1]
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
    d, cfg, tensors = folders["B"]
    a, b = tokens(cfg, 75, 1), tokens(cfg, 30, 2)
    ra, rb = pf.forward(cfg, tensors, a).numpy(), pf.forward(cfg, tensors, b).numpy()
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


def test_command_line_generates(folders, tmp_path):
    """`python -m sonicboom_b200 generate` on a Mefupel folder: greedy tokens as the plain
    implementation's, and a run with a repeat penalty (the loop on the host, no captured step)."""
    import subprocess
    import sys
    from conftest import ROOT
    d, cfg, tensors = folders["A"]
    prompts = [tokens(cfg, n, 50 + n) for n in (7, 33)]
    f = tmp_path / "prompts.txt"
    f.write_text("".join(" ".join(map(str, p)) + "\n" for p in prompts))
    base = [sys.executable, "-m", "sonicboom_b200", "generate", "-m", str(d), "--tokens", str(f), "-n", "6",
            "--dtype", "float32"]
    r = subprocess.run(base, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert got == [pf.greedy_generate(cfg, tensors, p, 6) for p in prompts]
    r = subprocess.run(base + ["--repeat-penalty", "1.5"], capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    penalized = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert [len(x) for x in penalized] == [6, 6]
