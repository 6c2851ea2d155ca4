"""Venadra (lightning attention with a decay per head, chunked attention with a sink, a short convolution in front of every
mixer, PolyNorm and softmax-routed gated experts, looped layers) on the GPU engine against the plain oracle of
tests/venadra_oracle.py: every mechanism alone, then whole models under every way of feeding them."""
import math
import random

import pytest
import torch

import venadra_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 0.15
PAGE = 32
F64 = torch.float64


def _light(heads=3, dim=24, vdim=40, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [0.35, 0.93, 0.9985, 1.0, 0.7][:heads]}


def _attn(heads=6, kv_heads=3, dim=24, vdim=40, size=37, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 3.0 / dim}
    if size:
        m["mask"] = {"size": size}
    return m


def _dense(ff=120):
    return {"kind": "dense", "ff": ff}


def _moe(experts=7, top=3, ff=40, limit=0.8, scale=1.3):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "scale": scale}}


def _cfg_a():
    """Sizes unlike powers of two: width 88, 5 taps; lightning heads 24 x 40 with a decay of exactly 1 among them;
    attention with 6 / 3 heads, keys of 24 and values of 40, chunks of 37 (no multiple of the page); one attention
    layer with keys as wide as values (the tensor-core kernel in bf16) in chunks of 64; a layer without feed-forward;
    layers 4 and 5 run the weights of layers 1 and 0."""
    return {"architecture": "Venadra", "width": 88, "vocab": 277, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
            "canon": {"taps": 5}, "layers": [
                {"type": "lightning", "mixer": _light(heads=4), "mlp": _dense()},
                {"type": "attention", "mixer": _attn(), "mlp": _moe()},
                {"type": "attention", "mixer": _attn(heads=4, kv_heads=1, dim=32, vdim=32, size=64), "mlp": None},
                {"type": "lightning", "mixer": _light(heads=1, dim=70, vdim=8, decay=[0.97]), "mlp": _moe(experts=3, top=1, ff=24, limit=2.0, scale=0.7)},
                {"type": "attention", "mixer": _attn(), "mlp": _moe(), "weights_of": 1},
                {"type": "lightning", "mixer": _light(heads=4), "mlp": _dense(), "weights_of": 0},
            ]}


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    from dllama_b200.models.layered import write_random_model
    d = str(tmp_path_factory.mktemp("venadra") / "a")
    cfg = _cfg_a()
    tensors = write_random_model(d, cfg, seed=3)
    g = torch.Generator().manual_seed(4)
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (150, 70, 5, 33)]
    want = [O.model_logits(tensors, cfg, r) for r in reqs]
    return d, cfg, tensors, reqs, want


def _engine(path, dtype="float32", max_rows=256, n_slots=4, seq=256, n_pages=None, **kw):
    from dllama_b200.models import registry
    return registry.engine_for_dir(path, max_rows=max_rows, n_slots=n_slots, max_seq_len=seq, n_pages=n_pages, dtype=dtype, **kw)


def _replay(eng, reqs, steps, free_when_done=True):
    fed, slot, got = {}, {}, {i: [] for i in range(len(reqs))}
    for step in steps:
        toks, pos, slots, owner = [], [], [], []
        for i, n in step:
            if i not in slot:
                slot[i], fed[i] = eng.alloc_slot(), 0
            toks += reqs[i][fed[i]:fed[i] + n]
            pos += list(range(fed[i], fed[i] + n))
            slots += [slot[i]] * n
            owner += [i] * n
            fed[i] += n
        lg = eng.forward(toks, pos, slots).cpu()
        for r, i in enumerate(owner):
            got[i].append(lg[r])
        for i, _ in step:
            if free_when_done and fed[i] == len(reqs[i]) and i in slot:
                eng.free_slot(slot.pop(i))
    return {i: torch.stack(v) for i, v in got.items() if v}


def _assert_close(got, want, tol, what="", flips=False):
    """flips: a bf16 run against the exact oracle.  Operand rounding moves router scores a little, and a token whose last
    chosen and first unchosen expert are closer than that takes another expert than the oracle and lands far off, with
    the tokens that read it.  So bf16 runs are held to the oracle in the bulk and, row by row and tightly, to the bf16
    run of the whole prompt (_assert_same); row-by-row exactness against the oracle is the f32 runs' part."""
    err = O.logit_error(got, want[:got.shape[0]])
    assert float(err.median()) < tol / 4, f"{what}: median error {float(err.median()):.3e}"
    if flips:
        over = int((err > tol).sum())
        assert over <= max(2, got.shape[0] // 4), f"{what}: {over} of {got.shape[0]} rows over {tol}"
    else:
        assert float(err.max()) < tol, f"{what}: worst row {int(err.argmax())} error {float(err.max()):.3e}"


def _assert_same(got, ref, what, tol=0.02):
    err = O.logit_error(got, ref[:got.shape[0]])
    over = int((err > tol).sum())
    assert over <= got.shape[0] // 50, f"{what}: {over} rows differ, worst row {int(err.argmax())} by {float(err.max()):.3e}"


# ---------------------------------------------------------------------------------------------------------------------
# a batch of rows for the kernels that walk sequences (the engine's descriptor, built by hand)
# ---------------------------------------------------------------------------------------------------------------------
class _Batch:
    """parts: [(slot, first position, rows)] in batch order; the rows of a part are consecutive."""

    def __init__(self, parts):
        from dllama_b200.ops import layers as L
        pos, row_seq, seq_start, seq_rows, seq_slot, seq_pos0, slots = [], [], [0], [], [], [], []
        for n, (slot, p0, rows) in enumerate(parts):
            seq_rows += list(range(len(pos), len(pos) + rows))
            pos += list(range(p0, p0 + rows))
            row_seq += [n] * rows
            slots += [slot] * rows
            seq_start.append(len(pos))
            seq_slot.append(slot)
            seq_pos0.append(p0)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
        self.pos, self.slot = i32(pos), i32(slots)
        self.keep = [self.pos, i32(row_seq), i32(seq_start), i32(seq_rows), i32(seq_slot), i32(seq_pos0)]
        self.desc = L.mamba_batch(*self.keep)
        self.M, self.n_seq, self.longest = len(pos), len(parts), max(r for _, _, r in parts)


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("taps,channels,wdtype", [(1, 40, torch.float32), (2, 333, torch.float32), (4, 96, torch.bfloat16), (9, 70, torch.float32)])
def test_input_convolution_carries_the_last_inputs_across_portions(taps, channels, wdtype):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(taps)
    T = 41
    seqs = [torch.randn(T, channels, generator=g), torch.randn(T, channels, generator=g)]
    w = (torch.randn(channels, taps, generator=g) * 0.5).to(wdtype)
    want = [O.short_convolution(s.double(), w.double()) for s in seqs]
    state = torch.randn(3, max(taps - 1, 1), channels, device="cuda")               # garbage of earlier users of the slots
    got = [[], []]
    at = [0, 0]
    # portions of 1, 2, taps - 1, ... rows, two sequences side by side in slots 2 and 0, unequal cuts
    for cut in ([(0, 1), (1, 3)], [(0, 2), (1, 1)], [(1, 2)], [(0, max(taps - 1, 1)), (1, 7)], [(0, 20), (1, 1)], [(0, 50), (1, 50)]):
        parts, xs = [], []
        for i, n in cut:
            n = min(n, T - at[i])
            if n:
                parts.append((2 if i == 0 else 0, at[i], n, i))
                xs.append(seqs[i][at[i]:at[i] + n])
        b = _Batch([(s, p, n) for s, p, n, _ in parts])
        x = torch.cat(xs).cuda().contiguous()
        out = torch.zeros_like(x)
        L.causal_conv(b.desc, b.M, b.n_seq, x, w.cuda(), state, out, residual=True)
        r = 0
        for s, p, n, i in parts:
            got[i].append(out[r:r + n].cpu())
            at[i] += n
            r += n
    for i in range(2):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=1e-5, rtol=1e-5), f"sequence {i}"


@pytest.mark.parametrize("dim", [40, 1000, 4500])
def test_poly_norm(dim):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(dim)
    z = torch.randn(5, dim, generator=g) * 2.0
    coef = torch.tensor([0.7, -0.3, 0.2, 0.05])
    a, b, c, e = coef.double()
    want = a * O.unit(z.double(), 1e-5) + b * O.unit(z.double() ** 2, 1e-5) + c * O.unit(z.double() ** 3, 1e-5) + e
    x = z.cuda()
    y = torch.zeros_like(x)
    L.poly_norm(x, y, 5, dim, coef.cuda(), 1e-5)
    assert torch.allclose(y.cpu().double(), want, atol=2e-5, rtol=2e-5)
    L.poly_norm(x, x, 5, dim, coef.cuda(), 1e-5)                                    # in place
    assert torch.equal(x, y)


@pytest.mark.parametrize("H,dim,vdim", [(2, 16, 16), (3, 24, 40), (1, 70, 8), (2, 128, 128), (1, 33, 150)])
def test_lightning_state_token_by_token_and_in_chunks(H, dim, vdim):
    """Three sequences of unequal length in one batch, fed in portions; the chunk-parallel form (portions of more than
    one chunk, with a ragged last chunk) and the token-by-token form leave the same state and outputs as the oracle.
    Decays from 0.05 (dies within a chunk) to exactly 1."""
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(H * 1000 + dim)
    lens = [300, 131, 64]
    decay = [0.05, 0.9, 1.0][:H] if H < 3 else [0.05, 0.995, 1.0]
    q = [torch.randn(n, H, dim, generator=g) * 0.4 for n in lens]
    k = [torch.randn(n, H, dim, generator=g) * 0.4 for n in lens]
    v = [torch.randn(n, H, vdim, generator=g) for n in lens]
    want = [torch.stack([O.decayed_linear_attention(q[i][:, h].double(), k[i][:, h].double(), v[i][:, h].double(), decay[h])
                         for h in range(H)], 1) for i in range(3)]
    dec = torch.tensor(decay, dtype=torch.float32, device="cuda")
    for chunked in (False, True):
        state = torch.randn(4, H, dim, vdim, device="cuda")                           # what earlier users left in the slots
        scratch = torch.zeros(L.lightning_chunk_floats(512, 3, H, dim, vdim), device="cuda")
        at, got = [0, 0, 0], [[], [], []]
        for cut in ([(0, 130), (1, 2), (2, 64)], [(0, 1), (1, 129)], [(0, 169)]):
            parts = [(3 - i, at[i], n, i) for i, n in cut]
            b = _Batch([(s, p, n) for s, p, n, _ in parts])
            cat = lambda xs: torch.cat([xs[i][at[i]:at[i] + n].reshape(n, -1) for _, _, n, i in parts]).cuda().contiguous()
            qq, kk, vv = cat(q), cat(k), cat(v)
            y = torch.zeros(b.M, H * vdim, device="cuda")
            use = chunked and L.lightning_chunked_supported(dim, vdim)
            L.lightning_scan(b.desc, b.n_seq, qq, kk, vv, dec, y, state, H, dim, vdim,
                             max_chunks=(b.longest + L.LIGHTNING_CHUNK - 1) // L.LIGHTNING_CHUNK if use else 0, scratch=scratch)
            r = 0
            for s, p, n, i in parts:
                got[i].append(y[r:r + n].cpu())
                at[i] += n
                r += n
        for i in range(3):
            out = torch.cat(got[i]).double().reshape(lens[i], H, vdim)
            scale = float(want[i].abs().max())
            assert float((out - want[i]).abs().max()) < 2e-5 * scale, (chunked, i, float((out - want[i]).abs().max()), scale)


def _attention_rows(q, k, v, scale, block, sink, ctype, tc=False, portions=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] through the cache writer (with the unit norms) and an attention kernel."""
    from dllama_b200.ops import layers as L
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    n_pages = (T + PAGE - 1) // PAGE
    cache = torch.zeros(n_pages + 2, G, PAGE, d + dv, dtype=ctype, device="cuda")
    table = torch.tensor([[0] * n_pages, list(range(n_pages + 1, 1, -1))], dtype=torch.int32, device="cuda")     # slot 1: pages in reverse
    out = []
    for p0, n in portions or [(0, T)]:
        pos = torch.arange(p0, p0 + n, dtype=torch.int32, device="cuda")
        slot = torch.ones(n, dtype=torch.int32, device="cuda")
        qq = q[p0:p0 + n].reshape(n, -1).float().cuda().contiguous()
        kk, vv = k[p0:p0 + n].reshape(n, -1).float().cuda().contiguous(), v[p0:p0 + n].reshape(n, -1).float().cuda().contiguous()
        freqs = torch.zeros(1, dtype=torch.float64, device="cuda")
        L.window_kv_write(kk, n, G, d, 0, freqs, 1.0, pos, slot, table, cache, q=qq, q_heads=H, v=vv, vdim=dv, qk_norm=True, eps=1e-5)
        o = torch.zeros(n, H * dv, device="cuda")
        sk = sink.float().cuda()
        if tc:
            rq = L.window_tc_rows(H, G)
            tiles = [list(range(i, min(i + rq, n))) for i in range(0, n, rq)]
            L.window_attention_tiles(qq, o, H, G, d, 0, scale, 0.0, 0, pos, slot, table, cache, tiles, n_splits=3 if n <= 2 * rq else 1,
                                     vdim=dv, chunk=block, sink=sk)
        else:
            L.window_attention(qq, o, n, H, G, d, 0, scale, 0.0, 0, pos, slot, table, cache, vdim=dv, chunk=block, sink=sk)
        out.append(o.cpu())
    return torch.cat(out).double().reshape(T, H, dv)


def _standout_case(block, T, H, G, d, dv, seed):
    """Keys that make one score stand out: for chosen queries i, key j(i) is the query's own direction, j(i) being the
    first position of i's block, the last of the block before it, or a far one -- a kernel that sees one key too many or
    too few returns another value than the oracle, not a slightly different one."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g) * 0.3, torch.randn(T, G, dv, generator=g)
    rep = H // G
    for i in range(block, T, 3):
        first = (i // block) * block
        j = (first, first - 1, max(first - block - 5, 0), i)[(i // 3) % 4]
        k[j] = q[i, ::rep][:G] * (1.0 if j != i else 0.9)
    return q, k, v


@pytest.mark.parametrize("ctype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block,H,G,d,dv", [(37, 6, 3, 24, 40), (32, 2, 2, 16, 16), (5, 4, 1, 32, 8), (0, 3, 1, 20, 20), (90, 10, 1, 16, 24)])
def test_chunked_attention_sees_exactly_its_chunk(ctype, block, H, G, d, dv):
    T = 150
    q, k, v = _standout_case(block or 50, T, H, G, d, dv, seed=block + H)
    sink = torch.linspace(-2.0, 3.0, H)
    scale = 12.0 / d
    # a bf16 cache holds the unit keys and the values rounded: small next to what one key too many or too few does
    rv = v if ctype == torch.float32 else v.bfloat16().float()
    want = O.block_sink_softmax_rows(q.double(), k.double(), rv.double(), scale, block, sink.double(), 1e-5)
    tol = 2e-4 if ctype == torch.float32 else 0.2
    for portions in (None, [(0, 36), (36, 2), (38, 1), (39, 59), (98, 52)]):
        got = _attention_rows(q, k, v, scale, block, sink, ctype, portions=portions)
        assert float((got - want).abs().max()) < tol, (portions, float((got - want).abs().max()))


@pytest.mark.parametrize("block,H,G,d", [(37, 6, 3, 32), (64, 4, 1, 64), (0, 8, 8, 16), (33, 2, 1, 128), (7, 5, 5, 48)])
def test_chunked_attention_on_the_tensor_cores_sees_exactly_its_chunk(block, H, G, d):
    from dllama_b200.ops import layers as L
    assert L.window_tc_supported(H, G, d, 0, torch.bfloat16)
    T = 200
    q, k, v = _standout_case(block or 50, T, H, G, d, d, seed=block + d)
    sink = torch.linspace(-1.0, 4.0, H)
    scale = 12.0 / d
    # what the kernel works on: unit keys rounded to bf16, values rounded to bf16; the queries are rounded after the norm
    want = O.block_sink_softmax_rows(q.double(), k.double(), v.bfloat16().double(), scale, block, sink.double(), 1e-5)
    for portions in (None, [(0, 36), (36, 2), (38, 1), (39, 59), (98, 102)]):          # short portions share their pages among CTAs
        got = _attention_rows(q, k, v, scale, block, sink, torch.bfloat16, tc=True, portions=portions)
        assert float((got - want).abs().max()) < 0.2, (portions, float((got - want).abs().max()))


def test_the_sink_takes_its_share_of_the_weights():
    """One visible key with score 0 and a sink of ln 3: the value comes out divided by 4."""
    q, k, v = torch.zeros(1, 2, 16), torch.zeros(1, 1, 16), torch.ones(1, 1, 16)
    sink = torch.tensor([math.log(3.0), -50.0])
    got = _attention_rows(q, k, v, 1.0, 8, sink, torch.float32)
    assert torch.allclose(got[0, 0], torch.full((16,), 0.25, dtype=F64), atol=1e-6)
    assert torch.allclose(got[0, 1], torch.ones(16, dtype=F64), atol=1e-6)


@pytest.mark.parametrize("E,top,scale", [(7, 3, 1.3), (12, 12, 1.0), (5, 1, 0.5), (64, 6, 2.0), (3, 2, 1.0), (40, 33, 1.5)])
def test_softmax_routing_renormalises_the_chosen_scores(E, top, scale):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(E * 10 + top)
    M = 50
    z = torch.randn(M, E, generator=g) * 3.0
    sel = torch.zeros(M, top, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(M, top, device="cuda")
    L.moe_select(z.cuda(), M, E, top, 1, 1, sel, wgt, renorm=True, softmax=True, scale=scale)
    for m in range(M):
        want = O.route(z[m].double(), {"experts": E, "top": top, "scale": scale})
        assert sel[m].tolist() == [e for e, _ in want], m
        assert torch.allclose(wgt[m].cpu().double(), torch.tensor([w for _, w in want], dtype=F64), atol=1e-6, rtol=1e-5)
        if top == E:
            assert abs(float(wgt[m].sum()) - scale) < 1e-5


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,W,ff,E,top,limit", [(1, 88, 40, 5, 2, 0.8), (7, 72, 24, 4, 4, 5.0), (70, 160, 56, 12, 3, 0.5), (300, 288, 100, 8, 3, 1.0)])
def test_gated_expert_products_both_forms(wdtype, M, W, ff, E, top, limit):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(M)
    wt = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1]) * 1.5).to(wdtype)
    w_gate, w_up, w_down = wt(E, ff, W), wt(E, ff, W), wt(E, W, ff)
    x = torch.randn(M, W, generator=g)
    xr = x.bfloat16().float() if wdtype == torch.bfloat16 else x
    sel = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(M)]).to(torch.int32)
    wgt = torch.rand(M, top, generator=g)
    w = {}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = w_gate[e].double(), w_up[e].double(), w_down[e].double()
    want = torch.stack([sum(float(wgt[m, j]) * O.gated_expert(xr[m].double(), w, int(sel[m, j]), limit) for j in range(top)) for m in range(M)])
    c = lambda t: t.cuda().contiguous()
    act, y = torch.zeros(M * top, ff, device="cuda"), torch.zeros(M, W, device="cuda")
    L.moe_rows(c(w_up), c(w_down), c(x), M, top, c(sel), c(wgt), act, y, wdtype == torch.bfloat16, w_gate=c(w_gate), limit=limit)
    tol = 1e-4 if wdtype == torch.float32 else 0.03                                  # bf16: the activation is rounded before W_down
    assert float((y.cpu().double() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))
    if wdtype == torch.bfloat16:
        grouped = L.MoeGrouped(c(w_up), c(w_down), top, M, w_gate=c(w_gate), limit=limit)
        y2 = torch.zeros(M, W, device="cuda")
        grouped.run(c(x), M, c(sel), c(wgt), y2)
        assert float((y2.cpu().double() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))


# ---------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_match_the_oracle(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    got = _replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i}", flips=dtype == "bfloat16")


def test_residual_stream_after_every_layer(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    res = []
    O.model_logits(tensors, cfg, reqs[3], residual_out=res)
    eng.layer_probe = []
    s = eng.alloc_slot()
    lg = eng.forward(reqs[3], list(range(len(reqs[3]))), [s] * len(reqs[3])).cpu()
    assert len(eng.layer_probe) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(eng.layer_probe, res)):
        assert torch.allclose(a.double().cpu(), b, atol=3e-4, rtol=3e-4), f"after layer {i}"
    _assert_close(lg, want[3], F32_TOL, "probed run")


def test_a_looped_layer_may_come_before_the_layer_whose_weights_it_runs(tmp_path):
    from dllama_b200.models.layered import write_random_model
    cfg = _cfg_a()
    L0, L1 = cfg["layers"][0], cfg["layers"][1]
    cfg["layers"] = [{**L1, "weights_of": 2}, {**L0, "weights_of": 3}, L1, L0]
    cfg["canon"] = {"taps": 2}
    tensors = write_random_model(str(tmp_path / "m"), cfg, seed=13)
    assert "l0.mix.q" not in tensors and "l2.mix.sink" in tensors and "l3.mlp.act" in tensors and tensors["l2.norm1"].dim() == 0
    req = torch.randint(0, cfg["vocab"], (80,), generator=torch.Generator().manual_seed(3)).tolist()
    got = _replay(_engine(str(tmp_path / "m")), [req], [[(0, 33)], [(0, 7)], [(0, 40)]])
    _assert_close(got[0], O.model_logits(tensors, cfg, req), F32_TOL, "forward reference")


def test_prefill_then_token_by_token(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    steps = [[(0, 105)]] + [[(0, 1)]] * 45 + [[(1, 1)]] * 70          # chunk edges at 111, 128 and 148 pass under decoded tokens
    got = _replay(eng, reqs, steps)
    _assert_close(got[0], want[0], F32_TOL, "prompt + decoded")
    _assert_close(got[1], want[1], F32_TOL, "decoded from the start")


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_portions_of_every_size(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    bf = dtype == "bfloat16"
    whole = _replay(eng, reqs, [[(0, 150)], [(1, 70)]])
    sizes = [2, 30, 1, 31, 2, 2, 33, 3, 32, 5, 2, 7]                  # cuts before, at and after page borders and chunk edges
    assert sum(sizes) == 150
    for what, i, steps in (("portions", 0, [[(0, n)] for n in sizes]), ("two tokens at a time", 1, [[(1, 2)]] * 35),
                           ("portions of the chunk's size", 0, [[(0, 37)], [(0, 38)], [(0, 75)]]),
                           ("the first token alone", 0, [[(0, 1)], [(0, 149)]])):
        got = _replay(eng, reqs, steps)
        _assert_close(got[i], want[i], tol, what, flips=bf)
        _assert_same(got[i], whole[i], what, 0.02 if bf else 1e-4)


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_mixed_batches_equal_each_request_alone(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    steps = [[(0, 3), (2, 1)], [(0, 40), (1, 2), (2, 1)], [(1, 30), (0, 1), (2, 2)], [(0, 1), (1, 1), (2, 1), (3, 20)],
             [(3, 13), (0, 64), (1, 5)], [(0, 1), (1, 32)], [(0, 40)]]
    got = _replay(eng, reqs, steps)
    assert got[0].shape[0] == 150 and got[1].shape[0] == 70 and got[2].shape[0] == 5 and got[3].shape[0] == 33
    whole = _replay(eng, reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], tol, f"request {i} in mixed batches", flips=dtype == "bfloat16")
        _assert_same(got[i], whole[i], f"request {i} in mixed batches against alone", 0.02 if dtype == "bfloat16" else 1e-4)


def test_pages_and_slots_are_reused_cleanly(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, max_rows=160, n_slots=1, seq=160, n_pages=5)
    for order in ([0, 2, 1, 3, 0], [3, 1]):
        for i in order:
            n = len(reqs[i])
            got = _replay(eng, reqs, [[(i, n // 2)], [(i, n - n // 2)]] if n > 1 else [[(i, n)]])
            _assert_close(got[i], want[i], F32_TOL, f"request {i} after reuse")
    assert len(eng.pages.free_pages) == 5 and len(eng.pages.free_slots) == 1
    eng2 = _engine(path, "bfloat16", max_rows=80, n_slots=2, seq=160, n_pages=6)       # two live requests share a small pool
    got = _replay(eng2, reqs, [[(1, 20), (3, 33)], [(1, 50)], [(2, 5), (0, 64)], [(0, 64)], [(0, 22)]])
    whole = _replay(_engine(path, "bfloat16"), reqs, [[(i, len(r))] for i, r in enumerate(reqs)])
    for i in got:
        _assert_close(got[i], want[i], BF16_TOL, f"request {i} in the shared pool", flips=True)
        _assert_same(got[i], whole[i], f"request {i} in the shared pool against alone")


def test_long_decoding_and_long_portions(model_a):
    path, cfg, tensors, reqs, want = model_a
    g = torch.Generator().manual_seed(21)
    seq = torch.randint(0, cfg["vocab"], (420,), generator=g).tolist()
    ref = O.model_logits(tensors, cfg, seq)
    eng = _engine(path, max_rows=512, seq=512)
    got = _replay(eng, [seq], [[(0, 6)]] + [[(0, 1)]] * 224 + [[(0, 190)]])       # the last portion runs the chunk-parallel scan on a carried state
    _assert_close(got[0], ref, F32_TOL, "224 decoded tokens, then a long portion")
    got = _replay(eng, [seq], [[(0, 300)], [(0, 120)]])
    _assert_close(got[0], ref, F32_TOL, "two long portions")


def test_a_far_token_reaches_the_end_only_through_the_recurrent_layer(tmp_path):
    """One token far back is changed.  Chunked attention and the short convolution carry it a chunk per layer at most, so
    with attention layers alone the last logits stay; with one slowly decaying lightning layer they move -- in the engine
    as in the oracle."""
    from dllama_b200.models.layered import write_random_model
    for first, moves in (("attention", False), ("lightning", True)):
        mix = _attn(heads=2, kv_heads=1, dim=32, vdim=32, size=24) if first == "attention" else _light(heads=2, dim=16, vdim=16, decay=[0.999, 0.5])
        cfg = {"architecture": "Venadra", "width": 64, "vocab": 97, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
               "canon": {"taps": 3}, "layers": [
                   {"type": first, "mixer": mix, "mlp": _moe(4, 2, 32)},
                   {"type": "attention", "mixer": _attn(heads=2, kv_heads=2, dim=16, vdim=24, size=24), "mlp": _dense(96)}]}
        d = str(tmp_path / first)
        tensors = write_random_model(d, cfg, seed=5)
        g = torch.Generator().manual_seed(6)
        a = torch.randint(0, 97, (120,), generator=g).tolist()
        b = list(a)
        b[10] = (a[10] + 1) % 97
        eng = _engine(d)
        wa, wb = O.model_logits(tensors, cfg, a), O.model_logits(tensors, cfg, b)
        _assert_close(ga := _replay(eng, [a], [[(0, 120)]])[0], wa, F32_TOL, "a")
        _assert_close(gb := _replay(eng, [b], [[(0, 100)]] + [[(0, 1)]] * 20)[0], wb, F32_TOL, "b")
        diff = float((ga[-1] - gb[-1]).abs().max())
        assert (diff > 1e-3) == moves, (first, diff)
        assert (float((wa[-1] - wb[-1]).abs().max()) > 1e-3) == moves


def test_greedy_generation_through_the_batching_loop(model_a, tmp_path):
    """The framework's own entry point: requests submitted to BatchEngine, batches formed by the C++ scheduler (prompt
    portions of 16 rows beside decoding rows), device greedy pick."""
    from dllama_b200.formats import tfile
    from dllama_b200.serving.batch_engine import BatchEngine, GenerationRequest
    from dllama_b200.text import native as T
    path, cfg, tensors, reqs, want = model_a
    tp = str(tmp_path / "t.t")
    tfile.write_synthetic_tokenizer(tp, cfg["vocab"])
    tok = T.Tokenizer(tp)
    eng = _engine(path, max_rows=32, n_slots=3, seq=128)
    be = BatchEngine(eng, tok, prefill_chunk=16)
    prompts = [reqs[1][:40], reqs[2], reqs[3][:20], reqs[0][:7], reqs[0][50:53]]
    n_new = 6
    rs = [be.submit(GenerationRequest(prompt_tokens=p, max_tokens=n_new, temperature=0.0)) for p in prompts]
    be.start()
    for r in rs:
        r.result(timeout=120)
    be.stop()
    assert be.n_errors == 0
    for r, p in zip(rs, prompts):
        seq = list(p)
        for _ in range(len(r.tokens)):
            seq.append(int(O.model_logits(tensors, cfg, seq)[-1].argmax()))
        assert r.tokens == seq[len(p):], (p, r.tokens, seq[len(p):])
        assert len(r.tokens) == n_new or tok.is_eos(r.tokens[-1])
    assert be.sched.stats()["free_slots"] == 3


def test_the_command_line_serves_the_model_directory(model_a):
    from dllama_b200.cli.app import build_engine
    from dllama_b200.ops import quant
    path, cfg, tensors, reqs, want = model_a
    eng = build_engine(path, 0, 1, 64, 2, 128, quant.F32, "cuda", dtype="float32")
    assert type(eng).__name__ == "LayerListEngine" and eng.h.vocab_size == cfg["vocab"] and eng.cfg.canon_taps == 5
    s = eng.alloc_slot()
    lg = eng.prefill(s, reqs[2])
    _assert_close(lg.cpu(), want[2][-1:], F32_TOL, "prefill() of the engine surface")


# ---------------------------------------------------------------------------------------------------------------------
# random configurations: sizes, layer lists and schedules drawn from a seed (f32, row by row against the oracle)
# ---------------------------------------------------------------------------------------------------------------------
def _random_config(rng):
    import json
    layers = []
    for i in range(rng.randint(1, 5)):
        own = [j for j in range(i) if "weights_of" not in layers[j]]
        if own and rng.random() < 0.3:
            j = rng.choice(own)
            layers.append({**json.loads(json.dumps(layers[j])), "weights_of": j})
            continue
        if rng.random() < 0.5:
            H = rng.choice([1, 2, 3, 5])
            kind, m = "lightning", _light(heads=H, dim=rng.choice([8, 16, 24, 48, 64, 100]), vdim=rng.choice([8, 16, 40, 64, 72, 128]),
                                           decay=[rng.choice([1.0, 0.9995, 0.97, 0.8, 0.3, 0.55]) for _ in range(H)])
        else:
            G, rep = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 5, 8])
            dim = rng.choice([16, 24, 48, 64, 80, 96, 128])
            kind, m = "attention", _attn(heads=G * rep, kv_heads=G, dim=dim, vdim=rng.choice([dim, dim, 8, 40, 72]),
                                           size=rng.choice([0, 1, 2, 7, 31, 32, 33, 65, 100]), scale=rng.choice([0.05, 0.15, 0.4]))
        mlp = None
        r = rng.random()
        if r < 0.45:
            E = rng.choice([1, 2, 5, 9, 16])
            mlp = _moe(experts=E, top=rng.randint(1, E), ff=rng.choice([16, 40, 130]), limit=rng.choice([0.5, 1.0, 7.0]), scale=rng.choice([1.0, 1.5, 0.3]))
        elif r < 0.9:
            mlp = _dense(rng.choice([24, 100, 256]))
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Venadra", "width": rng.choice([64, 100, 136, 192]), "vocab": rng.choice([97, 300, 513]),
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "embedding": {"scale": rng.choice([1.0, 2.5, 12.0])},
            "canon": {"taps": rng.choice([1, 2, 3, 4, 6])}, "layers": layers}


def _random_schedule(rng, lens):
    left, steps, live, pending = list(lens), [], [], list(range(len(lens)))
    while pending or live:
        while pending and len(live) < 3 and (not live or rng.random() < 0.7):
            live.append(pending.pop(0))
        step = []
        for i in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                                # a request sits a step out
            n = min(left[i], rng.choice([1, 1, 1, 2, 3, 17, 32, 33, 64, 90, 150]))
            step.append((i, n))
            left[i] -= n
            if left[i] == 0:
                live.remove(i)
        if step:
            steps.append(step)
    return steps


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 4, 5, 6, 7])
def test_random_configurations_and_schedules(tmp_path, seed):
    from dllama_b200.models.layered import write_random_model
    rng = random.Random(seed)
    cfg = _random_config(rng)
    tensors = write_random_model(str(tmp_path / "m"), cfg, seed=seed)
    g = torch.Generator().manual_seed(seed)
    lens = [rng.choice([1, 5, 40, 70, 130, 210]) for _ in range(4)]
    reqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lens]
    want = [O.model_logits(tensors, cfg, r) for r in reqs]
    n_pages = 3 * (max(lens) + 64) // PAGE
    eng = _engine(str(tmp_path / "m"), max_rows=n_pages * PAGE, n_slots=3, seq=n_pages * PAGE, n_pages=n_pages)
    got = _replay(eng, reqs, _random_schedule(rng, lens))
    for i in got:
        assert got[i].shape[0] == lens[i]
        _assert_close(got[i], want[i], F32_TOL, f"seed {seed}, request {i}: {cfg['layers']}")
    assert len(eng.pages.free_pages) == n_pages and len(eng.pages.free_slots) == 3
    eng.close()
    # the same model in bf16: fed in the schedule or whole, a row comes out the same
    eng = _engine(str(tmp_path / "m"), "bfloat16", max_rows=n_pages * PAGE, n_slots=3, seq=n_pages * PAGE, n_pages=n_pages)
    got = _replay(eng, reqs, _random_schedule(random.Random(seed + 100), lens))
    whole = _replay(eng, reqs, [[(i, n)] for i, n in enumerate(lens)])
    for i in got:
        _assert_same(got[i], whole[i], f"seed {seed}, request {i} in bf16", tol=0.03)
