"""Darusun (post-norm layers; grouped-query attention with rotate-half rotary, unit queries and keys and head-mixed
scores; latent attention with a sliding window, sinks and a gate per head; xIELU; experts with a router bias and a shared
expert) on the GPU engine against the plain oracle of tests/darusun_oracle.py: every mechanism alone, then whole models
under every way of feeding them."""
import json
import math
import random

import pytest
import torch

import darusun_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL, BF16_TOL = 2e-4, 0.15
PAGE = 32
F64 = torch.float64


def _attn(heads=6, kv_heads=3, dim=24, vdim=40, rot=16, scale=None, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 4.0 / dim, "rot": {"base": base, "dims": rot}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _latent(heads=3, dim=20, rot=8, vdim=28, q_rank=36, kv_rank=40, size=37, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale or 1.0 / math.sqrt(dim + rot), "rot": {"base": 5000.0, "dims": rot}}
    if size:
        m["mask"] = {"size": size}
    return m


def _dense(ff=120):
    return {"kind": "dense", "ff": ff}


def _moe(experts=7, top=3, ff=40, shared=56):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _cfg_a():
    """Sizes unlike powers of two: width 88; attention with 6 / 3 heads, keys of 24 (16 of them rotated) and values of 40;
    a latent layer with a window of 37 (no multiple of the page); a layer that reads layer 0's keys and values and whose
    experts all run; a layer with as many key/value heads as heads, rotary on the whole head and no feed-forward; a latent
    layer without a window; one key/value head and narrow values with a single expert per token."""
    return {"architecture": "Darusun", "width": 88, "vocab": 277, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "layers": [
        {"type": "attention", "mixer": _attn(), "mlp": _dense()},
        {"type": "latent_attention", "mixer": _latent(), "mlp": _moe()},
        {"type": "attention", "mixer": _attn(kv_from=0), "mlp": _moe(experts=5, top=5, ff=24, shared=0)},
        {"type": "attention", "mixer": _attn(heads=4, kv_heads=4, dim=32, vdim=32, rot=32), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(heads=2, dim=16, rot=16, vdim=16, q_rank=24, kv_rank=32, size=0), "mlp": _dense(64)},
        {"type": "attention", "mixer": _attn(heads=4, kv_heads=1, dim=16, vdim=8, rot=8), "mlp": _moe(experts=3, top=1, ff=24, shared=16)},
    ]}


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    from dllama_b200.models.layered import write_random_model
    d = str(tmp_path_factory.mktemp("darusun") / "a")
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
    """flips: a bf16 run against the exact oracle.  Operand rounding moves router logits by about a hundredth; a token whose
    last chosen and first unchosen expert are closer than that takes another expert than the oracle and lands far off, with
    the tokens that attend to it.  So bf16 runs are held to the oracle in the bulk and, row by row and tightly, to the bf16
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
# mechanisms alone: head-mixed attention
# ---------------------------------------------------------------------------------------------------------------------
def _attention_rows(q, k, v, talk, scale, rot, base, ctype, tc=False, portions=None, n_splits=1, write_kv=True, cache=None, fold=True):
    """q [T, H, d], k [T, G, d], v [T, G, dv] as projected, through the cache writer (rotary, unit norms, the head mix folded
    into the queries) and an attention kernel; pages of the slot in reverse order in a pool whose other lines hold garbage."""
    from dllama_b200.models.layered import rotary_frequencies
    from dllama_b200.ops import layers as L
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    n_pages = (T + PAGE - 1) // PAGE
    if cache is None:
        cache = (torch.randn(n_pages + 2, G, PAGE, d + dv, device="cuda") * 50).to(ctype)
    table = torch.tensor([[0] * n_pages, list(range(n_pages + 1, 1, -1))], dtype=torch.int32, device="cuda")
    freqs = rotary_frequencies(base, rot).cuda() if rot else torch.zeros(1, dtype=torch.float64, device="cuda")
    tk = talk.float().cuda().contiguous()
    out = []
    for p0, n in portions or [(0, T)]:
        pos = torch.arange(p0, p0 + n, dtype=torch.int32, device="cuda")
        slot = torch.ones(n, dtype=torch.int32, device="cuda")
        qq = q[p0:p0 + n].reshape(n, -1).float().cuda().contiguous()
        kk, vv = k[p0:p0 + n].reshape(n, -1).float().cuda().contiguous(), v[p0:p0 + n].reshape(n, -1).float().cuda().contiguous()
        qm = torch.zeros(n, H * G * d, device="cuda")
        L.window_kv_write(kk if write_kv else None, n, G, d, rot, freqs, 1.0, pos, slot, table, cache, q=qq, q_heads=H,
                          v=vv if write_kv else None, vdim=dv, qk_norm=True, eps=1e-5, rope_half=True, talk=tk, q_mixed=qm)
        o = torch.zeros(n, H * dv, device="cuda")
        if tc:
            rq = L.talk_tc_rows(H, G, d, dv, G, n)          # tiles of 16, 64 or 128 stacked (row, head) pairs by the portion's length
            tiles = [list(range(i, min(i + rq, n))) for i in range(0, n, rq)]
            L.talk_attention_tiles(qm if fold else qq, o, H, G, d, dv, scale, 0, pos, slot, table, cache, tiles, rq, n_splits=n_splits,
                                   key_heads=G if fold else 0)
        else:
            L.window_attention(qm, o, n, H, G, d, 0, scale, 0.0, 0, pos, slot, table, cache, vdim=dv, key_heads=G)
        out.append(o.cpu())
    return torch.cat(out).double().reshape(T, H, dv), cache


def _mixed_case(T, H, G, d, dv, seed):
    """Random q, k, v and a head mix with real cross-talk.  For chosen queries one key far back (position 0, a page border,
    the query's own place, ...) is made the direction of one of the query's heads, so that one raw score stands out by e^12:
    a kernel that misses that key, or folds the mix wrongly, returns another value, not a slightly different one."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    talk = torch.eye(H) * 0.8 + torch.randn(H, H, generator=g) * 0.4
    rep = H // G
    places = [0, 1, 31, 32, 33, 63, 64]
    for n, i in enumerate(range(3, T, 5)):
        j = (places[n % len(places)], i, i - 1, max(i - 100, 0))[n % 4]
        if j <= i:
            h = n % H
            k[j, h // rep] = q[i, h] * 3.0
    return q, k, v, talk.bfloat16().float()


def _mixed_want(q, k, v, talk, scale, rot, base, eps=1e-5):
    T = q.shape[0]
    pos = torch.arange(T)
    qn = O.rms_unit(O.rotate_half_pairs(q.double(), pos, base, rot), eps) if rot else O.rms_unit(q.double(), eps)
    kn = O.rms_unit(O.rotate_half_pairs(k.double(), pos, base, rot), eps) if rot else O.rms_unit(k.double(), eps)
    return O.mixed_head_softmax_rows(qn, kn, v.double(), scale, talk.double()), qn, kn


@pytest.mark.parametrize("H,G,d,dv,rot", [(6, 3, 24, 40, 16), (4, 1, 32, 8, 32), (3, 3, 16, 16, 4), (8, 2, 64, 80, 32), (10, 1, 20, 24, 0), (2, 2, 9, 5, 6)])
def test_rotary_unit_norm_and_the_head_mix_folded_into_the_queries(H, G, d, dv, rot):
    """The writer alone: queries in place, keys in the cache, and the folded queries, whose products with the keys of all
    key/value heads side by side are the mixed scores."""
    from dllama_b200.models.layered import rotary_frequencies
    from dllama_b200.ops import layers as L
    T, base = 70, 3000.0
    q, k, v, talk = _mixed_case(T, H, G, d, dv, seed=H + d)
    cache = torch.zeros(4, G, PAGE, d + dv, device="cuda")
    table = torch.tensor([[3, 1, 2]], dtype=torch.int32, device="cuda")
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device="cuda")                  # positions 5 .. 74: rotary by the position, not the row
    turn = (lambda x: O.rotate_half_pairs(x.double(), pos.cpu(), base, rot)) if rot else (lambda x: x.double())
    qn, kn = O.rms_unit(turn(q), 1e-5), O.rms_unit(turn(k), 1e-5)
    slot = torch.zeros(T, dtype=torch.int32, device="cuda")
    qq, kk, vv = (t.reshape(T, -1).float().cuda().contiguous() for t in (q, k, v))
    qm = torch.zeros(T, H * G * d, device="cuda")
    freqs = rotary_frequencies(base, rot).cuda() if rot else torch.zeros(1, dtype=torch.float64, device="cuda")
    L.window_kv_write(kk, T, G, d, rot, freqs, 1.0, pos, slot, table, cache, q=qq, q_heads=H, v=vv, vdim=dv, qk_norm=True, eps=1e-5,
                      rope_half=True, talk=talk.cuda(), q_mixed=qm)
    assert torch.allclose(qq.cpu().double().reshape(T, H, d), qn, atol=2e-5)
    lines = torch.stack([cache[[3, 1, 2][p // PAGE], :, p % PAGE] for p in pos.tolist()]).cpu().double()      # [T, G, d + dv]
    assert torch.allclose(lines[..., :d], kn, atol=2e-5) and torch.allclose(lines[..., d:], v.double(), atol=1e-6)
    rep = H // G
    raw = torch.einsum("thd,shd->hts", qn, kn.repeat_interleave(rep, 1))               # raw scores of head h
    mixed = torch.einsum("hg,gts->hts", talk.double(), raw)
    folded = torch.einsum("thx,sx->hts", qm.cpu().double().reshape(T, H, G * d), kn.reshape(T, G * d))
    assert torch.allclose(folded, mixed, atol=1e-4)


@pytest.mark.parametrize("ctype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,rot", [(6, 3, 24, 40, 16), (4, 1, 32, 8, 32), (3, 3, 16, 16, 4), (8, 2, 64, 80, 32), (10, 1, 20, 24, 0), (2, 2, 9, 5, 6)])
def test_head_mixed_attention_sees_every_key_up_to_its_position(ctype, H, G, d, dv, rot):
    T, scale = 150, 12.0 / d
    q, k, v, talk = _mixed_case(T, H, G, d, dv, seed=H * 7 + d)
    rv = v if ctype == torch.float32 else v.bfloat16().float()
    want, _, _ = _mixed_want(q, k, rv, talk, scale, rot, 20000.0)
    tol = 3e-4 if ctype == torch.float32 else 0.25           # a bf16 cache rounds the unit keys: small next to one key too many or too few
    for portions in (None, [(0, 36), (36, 2), (38, 1), (39, 59), (98, 52)], [(0, 149), (149, 1)]):
        got, _ = _attention_rows(q, k, v, talk, scale, rot, 20000.0, ctype, portions=portions)
        assert float((got - want).abs().max()) < tol, (portions, float((got - want).abs().max()))


@pytest.mark.parametrize("H,G,d,dv,rot", [(6, 3, 24, 40, 16), (6, 2, 64, 80, 32), (4, 4, 32, 32, 32), (8, 1, 128, 128, 64), (2, 2, 16, 8, 0), (5, 1, 40, 104, 8), (16, 4, 128, 128, 64)])
def test_head_mixed_attention_on_the_tensor_cores(H, G, d, dv, rot):
    from dllama_b200.ops import layers as L
    assert L.talk_tc_supported(H, G, d, dv, G, torch.bfloat16)
    T, scale = 200, 12.0 / d
    q, k, v, talk = _mixed_case(T, H, G, d, dv, seed=H * 3 + dv)
    # what the kernel works on: unit keys and values rounded to bf16; the folded queries are rounded too
    want, _, _ = _mixed_want(q, k, v.bfloat16().float(), talk, scale, rot, 20000.0)
    for portions, n_splits in ((None, 1), ([(0, 36), (36, 2), (38, 1), (39, 59), (98, 102)], 3), ([(0, 199), (199, 1)], 16)):
        got, _ = _attention_rows(q, k, v, talk, scale, rot, 20000.0, torch.bfloat16, tc=True, portions=portions, n_splits=n_splits)
        assert float((got - want).abs().max()) < 0.25, (portions, float((got - want).abs().max()))


@pytest.mark.parametrize("H,G,d,dv,rot", [(6, 3, 24, 40, 16), (16, 4, 128, 128, 64), (8, 8, 32, 16, 0), (10, 2, 64, 80, 32)])
def test_many_decoding_rows_share_one_staging_of_all_heads(H, G, d, dv, rot):
    """Single rows of many sequences in one launch (here: 160 positions of one sequence as 160 one-row tiles with page
    shares): enough CTAs for the form in which one CTA serves every key/value head of its tile."""
    from dllama_b200.models.layered import rotary_frequencies
    from dllama_b200.ops import layers as L
    T, scale = 160, 12.0 / d
    q, k, v, talk = _mixed_case(T, H, G, d, dv, seed=H + G)
    want, _, _ = _mixed_want(q, k, v.bfloat16().float(), talk, scale, rot, 20000.0)
    n_pages = T // PAGE
    cache = (torch.randn(n_pages + 1, G, PAGE, d + dv, device="cuda") * 50).to(torch.bfloat16)
    table = torch.tensor([list(range(n_pages, 0, -1))], dtype=torch.int32, device="cuda")
    freqs = rotary_frequencies(20000.0, rot).cuda() if rot else torch.zeros(1, dtype=torch.float64, device="cuda")
    pos, slot = torch.arange(T, dtype=torch.int32, device="cuda"), torch.zeros(T, dtype=torch.int32, device="cuda")
    qq, kk, vv = (t.reshape(T, -1).float().cuda().contiguous() for t in (q, k, v))
    qm, o = torch.zeros(T, H * G * d, device="cuda"), torch.zeros(T, H * dv, device="cuda")
    L.window_kv_write(kk, T, G, d, rot, freqs, 1.0, pos, slot, table, cache, q=qq, q_heads=H, v=vv, vdim=dv, qk_norm=True, eps=1e-5,
                      rope_half=True, talk=talk.cuda(), q_mixed=qm)
    rq = L.talk_tc_rows(H, G, d, dv, G, 1)
    assert rq * (H // G) <= 16
    L.talk_attention_tiles(qm, o, H, G, d, dv, scale, 0, pos, slot, table, cache, [[i] for i in range(T)], rq, n_splits=4, key_heads=G)
    got = o.cpu().double().reshape(T, H, dv)
    assert float((got - want).abs().max()) < 0.25, float((got - want).abs().max())


@pytest.mark.parametrize("H,G,d,dv", [(6, 3, 24, 40), (8, 2, 64, 80), (4, 1, 32, 8), (16, 8, 16, 104)])
def test_the_tile_kernel_without_a_head_mix_is_plain_grouped_query_attention(H, G, d, dv):
    """key_heads = 0: every head meets its own group's key; values of another width than the keys."""
    T, scale = 130, 12.0 / d
    q, k, v, _ = _mixed_case(T, H, G, d, dv, seed=H + dv)
    eye = torch.eye(H)
    want, _, _ = _mixed_want(q, k, v.bfloat16().float(), eye, scale, 8, 20000.0)
    for portions, n_splits in ((None, 1), ([(0, 36), (36, 2), (38, 1), (39, 91)], 3), ([(0, 129), (129, 1)], 5)):
        got, _ = _attention_rows(q, k, v, eye, scale, 8, 20000.0, torch.bfloat16, tc=True, portions=portions, n_splits=n_splits, fold=False)
        assert float((got - want).abs().max()) < 0.25, (portions, float((got - want).abs().max()))


def test_a_layer_without_keys_of_its_own_reads_the_cache_it_is_given():
    H, G, d, dv, rot, T = 6, 3, 24, 40, 16, 90
    q, k, v, talk = _mixed_case(T, H, G, d, dv, seed=5)
    scale = 12.0 / d
    first, cache = _attention_rows(q, k, v, talk, scale, rot, 20000.0, torch.float32)
    g = torch.Generator().manual_seed(9)
    q2, talk2 = torch.randn(T, H, d, generator=g), torch.randn(H, H, generator=g)
    want, _, _ = _mixed_want(q2, k, v, talk2, scale, rot, 20000.0)
    before = cache.clone()
    got, _ = _attention_rows(q2, k * 0 + 7, v * 0 + 7, talk2, scale, rot, 20000.0, torch.float32, write_kv=False, cache=cache)
    assert torch.equal(cache, before)
    assert float((got - want).abs().max()) < 3e-4


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone: latent attention with a window, sinks and a gate per head
# ---------------------------------------------------------------------------------------------------------------------
def _latent_rows(q_lat, q_rot, c, kr, gate, sink, scale, size, ctype, tc=False, portions=None, n_splits=1):
    """q_lat [T, H, r] / q_rot [T, H, rot] against cache lines [c | kr] (written as they are), per-row or tile kernel."""
    from dllama_b200.ops import layers as L
    T, H, r = q_lat.shape
    rot = kr.shape[1]
    n_pages = (T + PAGE - 1) // PAGE
    cache = (torch.randn(n_pages + 2, PAGE, r + rot, device="cuda") * 50).to(ctype)
    order = list(range(n_pages + 1, 1, -1))
    for p in range(T):
        cache[order[p // PAGE], p % PAGE] = torch.cat([c[p], kr[p]]).to(ctype).cuda()
    table = torch.tensor([[0] * n_pages, order], dtype=torch.int32, device="cuda")
    out = []
    for p0, n in portions or [(0, T)]:
        pos = torch.arange(p0, p0 + n, dtype=torch.int32, device="cuda")
        slot = torch.ones(n, dtype=torch.int32, device="cuda")
        ql = q_lat[p0:p0 + n].reshape(n, H * r).float().cuda().contiguous()
        qr = q_rot[p0:p0 + n].reshape(n, H * rot).float().cuda().contiguous()
        gz = gate[p0:p0 + n].float().cuda().contiguous()
        o = torch.zeros(n, H * r, device="cuda")
        tiles = None
        if tc:
            rq = max(1, min(16, 64 // H)) if n > max(1, 32 // H) else max(1, min(16, 32 // H))
            assert L.latent_tc_supported(H, r, rot, ctype, rq)
            rows = [list(range(i, min(i + rq, n))) + [-1] * (rq - min(rq, n - i)) for i in range(0, n, rq)]
            part = torch.zeros(L.latent_tc_partial_floats(len(rows), n_splits, r), device="cuda")
            tiles = (torch.tensor(rows, dtype=torch.int32).cuda(), len(rows), rq, n_splits, part)
        L.latent_attention(ql, qr, rot, 0, o, n, H, r, rot, scale, pos, slot, table, cache, tiles=tiles, window=size,
                           sink=sink.float().cuda(), gate=gz)
        out.append(o.cpu())
    return torch.cat(out).double().reshape(T, H, r)


def _latent_case(T, H, r, rot, size, seed):
    """One cache line per chosen query is made the query's own direction: the line just inside the window (i - size + 1),
    just outside (i - size), at the query itself, or at a page border."""
    g = torch.Generator().manual_seed(seed)
    q_lat, q_rot = torch.randn(T, H, r, generator=g), torch.randn(T, H, rot, generator=g)
    c, kr = torch.randn(T, r, generator=g) * 0.3, torch.randn(T, rot, generator=g) * 0.3
    span = size or 70
    for n, i in enumerate(range(span, T, 3)):
        j = (i - span + 1, i - span, i, (i // PAGE) * PAGE - 1)[n % 4]
        c[j], kr[j] = q_lat[i, n % H], q_rot[i, n % H]
    gate = torch.randn(T, H, generator=g) * 2
    return q_lat, q_rot, c, kr, gate


def _latent_want(q_lat, q_rot, c, kr, gate, sink, scale, size):
    H = q_lat.shape[1]
    scores = (torch.einsum("ihr,jr->hij", q_lat.double(), c.double()) + torch.einsum("ihr,jr->hij", q_rot.double(), kr.double())) * scale
    o = O.window_sink_softmax_rows(scores, c.double()[:, None, :].expand(-1, H, -1), size, sink.double())
    return o * torch.sigmoid(gate.double())[:, :, None]


@pytest.mark.parametrize("ctype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,r,rot,size", [(3, 40, 8, 37), (2, 32, 16, 32), (5, 24, 8, 1), (4, 48, 16, 0), (1, 20, 4, 100), (8, 64, 8, 33)])
def test_latent_attention_sees_exactly_its_window(ctype, H, r, rot, size):
    T, scale = 170, 12.0 / (r + rot)
    q_lat, q_rot, c, kr, gate = _latent_case(T, H, r, rot, size, seed=H + r)
    sink = torch.linspace(-2.0, 3.0, H)
    rc, rk = (c, kr) if ctype == torch.float32 else (c.bfloat16().float(), kr.bfloat16().float())
    want = _latent_want(q_lat, q_rot, rc, rk, gate, sink, scale, size)
    tol = 3e-4 if ctype == torch.float32 else 0.05
    for portions in (None, [(0, 36), (36, 2), (38, 1), (39, 59), (98, 72)], [(0, 169), (169, 1)]):
        got = _latent_rows(q_lat, q_rot, c, kr, gate, sink, scale, size, ctype, portions=portions)
        assert float((got - want).abs().max()) < tol, (portions, float((got - want).abs().max()))


@pytest.mark.parametrize("H,r,rot,size", [(3, 40, 8, 37), (2, 32, 16, 32), (8, 128, 32, 96), (4, 48, 16, 0), (16, 24, 8, 5), (1, 64, 8, 100)])
def test_latent_attention_on_the_tensor_cores_sees_exactly_its_window(H, r, rot, size):
    T, scale = 200, 12.0 / (r + rot)
    q_lat, q_rot, c, kr, gate = _latent_case(T, H, r, rot, size, seed=H * 5 + r)
    sink = torch.linspace(-1.0, 4.0, H)
    want = _latent_want(q_lat, q_rot, c.bfloat16().float(), kr.bfloat16().float(), gate, sink, scale, size)
    for portions, n_splits in ((None, 1), ([(0, 36), (36, 2), (38, 1), (39, 59), (98, 102)], 3), ([(0, 199), (199, 1)], 7)):
        got = _latent_rows(q_lat, q_rot, c, kr, gate, sink, scale, size, torch.bfloat16, tc=True, portions=portions, n_splits=n_splits)
        assert float((got - want).abs().max()) < 0.3, (portions, n_splits, float((got - want).abs().max()))


def test_the_sink_and_the_gate_take_their_share():
    """One visible key of score 0 beside a sink of ln 3: the key gets a quarter of the weight; a gate of 0 halves it."""
    q_lat, q_rot = torch.zeros(1, 2, 16), torch.zeros(1, 2, 8)
    c, kr = torch.arange(16.0)[None, :], torch.zeros(1, 8)
    sink, gate = torch.tensor([math.log(3.0), -1e4]), torch.tensor([[0.0, 50.0]])
    for ctype, tc in ((torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)):
        got = _latent_rows(q_lat, q_rot, c, kr, gate, sink, 1.0, 5, ctype, tc=tc)
        assert torch.allclose(got[0, 0], c[0].double() / 8, atol=1e-5) and torch.allclose(got[0, 1], c[0].double(), atol=1e-5)


# ---------------------------------------------------------------------------------------------------------------------
# mechanisms alone: feed-forwards
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,K,N,wdtype", [(1, 88, 120, torch.float32), (7, 64, 33, torch.bfloat16), (40, 100, 72, torch.float32), (300, 160, 200, torch.bfloat16)])
def test_xielu_and_the_gated_epilogues_of_the_dense_products(M, K, N, wdtype):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(M + N)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(wdtype)
    x, aux, y0, row = torch.randn(M, K, generator=g) * 2, torch.randn(M, N, generator=g), torch.randn(M, N, generator=g), torch.randn(M, 1, generator=g)
    rx = wdtype == torch.bfloat16
    xd = (x.bfloat16() if rx else x).double()
    z = xd @ w.double().T
    p, q = 0.3, -0.7
    ap, bq = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
    want = {L.DENSE_XIELU: O.xielu(z, p, q), L.DENSE_MUL: aux.double() * z, L.DENSE_ROWGATE_ADD: y0.double() + torch.sigmoid(row.double()) * z}
    forms = ["stream"] + (["tc"] if rx and M >= 32 else [])
    for form in forms:
        for op, ref in want.items():
            y = y0.clone().cuda() if op == L.DENSE_ROWGATE_ADD else torch.zeros(M, N, device="cuda")
            a = {L.DENSE_XIELU: None, L.DENSE_MUL: aux.cuda(), L.DENSE_ROWGATE_ADD: row.cuda()}[op]
            if form == "tc":
                ncap = (M + 7) // 8 * 8
                xh = torch.zeros(L.xh_bytes(K, ncap), dtype=torch.uint8, device="cuda")
                L.xh_from_rows(x.cuda(), M, K, ncap, xh)
                L.dense_tc(L.make_wh(w.cuda()), N, K, xh, ncap, y, M, epi=op, aux=a, param=ap, param2=bq)
            else:
                L.dense(w.cuda(), x.cuda(), y, M, rx, epi=op, aux=a, param=ap, param2=bq)
            assert torch.allclose(y.cpu().double(), ref, atol=2e-4, rtol=2e-4), (form, op, float((y.cpu().double() - ref).abs().max()))


@pytest.mark.parametrize("E,top", [(7, 3), (12, 12), (5, 1), (64, 6), (3, 2), (40, 33), (1, 1)])
def test_routing_by_biased_logits_weighs_the_chosen_by_their_softmax(E, top):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(E)
    M = 50
    z, b = torch.randn(M, E, generator=g) * 3, torch.randn(E, generator=g) * 2
    if E > 3:
        b[2] = 6.0                     # a bias that decides: expert 2 is chosen almost always, whatever its logit
    sel, wgt = torch.zeros(M, top, dtype=torch.int32, device="cuda"), torch.zeros(M, top, device="cuda")
    L.moe_select(z.cuda(), M, E, top, 1, 1, sel, wgt, renorm=True, softmax=True, bias=b.cuda())
    ws, ww = O.route(z.double() + b.double(), top)
    assert torch.equal(sel.cpu().long(), ws)
    assert torch.allclose(wgt.cpu().double(), ww, atol=1e-6)


@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,W,ff,E,top", [(1, 88, 40, 5, 2), (7, 72, 24, 4, 4), (70, 160, 56, 12, 3), (300, 288, 100, 8, 3)])
def test_gated_silu_expert_products_both_forms(wdtype, M, W, ff, E, top):
    from dllama_b200.ops import layers as L
    g = torch.Generator().manual_seed(M + ff)
    mk = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(wdtype)
    wg, wu, wd = mk(E, ff, W), mk(E, ff, W), mk(E, W, ff)
    x = torch.randn(M, W, generator=g)
    sel = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(M)]).int()
    wgt = torch.rand(M, top, generator=g)
    rx = wdtype == torch.bfloat16
    xd = (x.bfloat16() if rx else x).double()
    want = torch.zeros(M, W, dtype=F64)
    for m in range(M):
        for k in range(top):
            e = int(sel[m, k])
            gg = xd[m] @ wg[e].double().T
            hid = gg * torch.sigmoid(gg) * (xd[m] @ wu[e].double().T)
            if rx:
                hid = hid.float().bfloat16().double()
            want[m] += float(wgt[m, k]) * (hid @ wd[e].double().T)
    act, y = torch.zeros(M * top, ff, device="cuda"), torch.zeros(M, W, device="cuda")
    L.moe_rows(wu.cuda(), wd.cuda(), x.cuda(), M, top, sel.cuda(), wgt.cuda(), act, y, rx, w_gate=wg.cuda(), gate_silu=True)
    assert torch.allclose(y.cpu().double(), want, atol=3e-3 if rx else 2e-4, rtol=1e-3)
    if rx and M >= 32:
        grp = L.MoeGrouped(wu.cuda(), wd.cuda(), top, M, w_gate=wg.cuda(), gate_silu=True)
        y2 = torch.zeros(M, W, device="cuda")
        grp.run(x.cuda(), M, sel.cuda(), wgt.cuda(), y2)
        assert torch.allclose(y2.cpu().double(), want, atol=3e-3, rtol=1e-3)


# ---------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_whole_prompts_match_the_oracle(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    if dtype == "bfloat16":          # the tile kernels are the ones that run
        assert eng.layers[0].mixer.tc_talk and eng.layers[2].mixer.tc_talk and eng.attn_rq
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


def test_prefill_then_token_by_token(model_a):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path)
    steps = [[(0, 105)]] + [[(0, 1)]] * 45 + [[(1, 1)]] * 70          # the window of 37 passes over decoded tokens; request 1 is decoded from its first token
    got = _replay(eng, reqs, steps)
    _assert_close(got[0], want[0], F32_TOL, "prompt + decoded")
    _assert_close(got[1], want[1], F32_TOL, "decoded from the start")


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_portions_of_every_size(model_a, dtype, tol):
    path, cfg, tensors, reqs, want = model_a
    eng = _engine(path, dtype)
    bf = dtype == "bfloat16"
    whole = _replay(eng, reqs, [[(0, 150)], [(1, 70)]])
    sizes = [2, 30, 1, 31, 2, 2, 33, 3, 32, 5, 2, 7]                  # cuts before, at and after page borders and the window's edge
    assert sum(sizes) == 150
    for what, i, steps in (("portions", 0, [[(0, n)] for n in sizes]), ("two tokens at a time", 1, [[(1, 2)]] * 35),
                           ("portions of the window's size", 0, [[(0, 37)], [(0, 38)], [(0, 75)]]),
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
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        eng = _engine(path, dtype, max_rows=512, seq=512)
        got = _replay(eng, [seq], [[(0, 6)]] + [[(0, 1)]] * 224 + [[(0, 190)]])
        _assert_close(got[0], ref, tol, "224 decoded tokens, then a long portion", flips=dtype == "bfloat16")
        got2 = _replay(eng, [seq], [[(0, 300)], [(0, 120)]])
        _assert_close(got2[0], ref, tol, "two long portions", flips=dtype == "bfloat16")
        _assert_same(got[0], got2[0], "decoded against portions", 0.02 if dtype == "bfloat16" else 1e-4)


def test_a_far_token_reaches_the_end_only_through_the_unwindowed_layer(tmp_path):
    """One token far back is changed.  Windowed latent layers carry it a window per layer at most, so with them alone the
    last logits stay; with one full attention layer they move -- in the engine as in the oracle."""
    from dllama_b200.models.layered import write_random_model
    for first, moves in (("latent_attention", False), ("attention", True)):
        mix = _latent(heads=2, dim=16, rot=8, vdim=16, q_rank=24, kv_rank=24, size=24) if first == "latent_attention" else _attn(heads=2, kv_heads=1, dim=16, vdim=24, rot=8)
        cfg = {"architecture": "Darusun", "width": 64, "vocab": 97, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "layers": [
            {"type": first, "mixer": mix, "mlp": _moe(4, 2, 32, 24)},
            {"type": "latent_attention", "mixer": _latent(heads=2, dim=8, rot=8, vdim=24, q_rank=16, kv_rank=24, size=24), "mlp": _dense(96)}]}
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
    assert type(eng).__name__ == "LayerListEngine" and eng.h.vocab_size == cfg["vocab"] and eng.cfg.residual == "post"
    s = eng.alloc_slot()
    lg = eng.prefill(s, reqs[2])
    _assert_close(lg.cpu(), want[2][-1:], F32_TOL, "prefill() of the engine surface")


# ---------------------------------------------------------------------------------------------------------------------
# random configurations: sizes, layer lists and schedules drawn from a seed (f32, row by row against the oracle)
# ---------------------------------------------------------------------------------------------------------------------
def _random_config(rng):
    layers = []
    for i in range(rng.randint(1, 5)):
        if rng.random() < 0.6:
            G, rep = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 5, 8])
            dim = rng.choice([16, 24, 36, 48, 64, 80, 128])
            m = _attn(heads=G * rep, kv_heads=G, dim=dim, vdim=rng.choice([dim, 8, 20, 40, 72, 128]), rot=rng.choice([dim, dim // 2, 4, 8]),
                      scale=rng.choice([0.05, 0.15, 0.4]), base=rng.choice([100.0, 10000.0, 500000.0]))
            same = [j for j in range(i) if layers[j]["type"] == "attention" and "kv_from" not in layers[j]["mixer"]]
            if same and rng.random() < 0.4:           # this layer's own queries and head mix on an earlier layer's keys and values
                j = rng.choice(same)
                m = {**json.loads(json.dumps(layers[j]["mixer"])), "scale": m["scale"], "kv_from": j}
            kind = "attention"
        else:
            rot = rng.choice([4, 8, 16, 32])
            kind, m = "latent_attention", _latent(heads=rng.choice([1, 2, 3, 5, 8]), dim=rng.choice([8, 16, 24, 40, 64]), rot=rot,
                                                  vdim=rng.choice([8, 16, 28, 64]), q_rank=rng.choice([16, 36, 64]),
                                                  kv_rank=rng.choice([16, 24, 40, 52, 64, 128]), size=rng.choice([0, 1, 2, 7, 31, 32, 33, 65, 100]))
        mlp = None
        r = rng.random()
        if r < 0.5:
            E = rng.choice([1, 2, 5, 9, 16])
            mlp = _moe(experts=E, top=rng.randint(1, E), ff=rng.choice([16, 40, 130]), shared=rng.choice([0, 8, 40, 100]))
        elif r < 0.9:
            mlp = _dense(rng.choice([24, 100, 256]))
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Darusun", "width": rng.choice([64, 100, 136, 192]), "vocab": rng.choice([97, 300, 513]),
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "residual_mult": rng.choice([1.0, 0.7, 0.3]), "layers": layers}


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
