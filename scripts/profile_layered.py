#!/usr/bin/env python3
"""Workloads for launch lists and counter captures of the layer-list models (one GPU).

  python scripts/profile_layered.py steps --design sunesun --size w2048
      one 2048-token prompt per slot, then decode steps of 1 and of 32 rows, launched eagerly (no CUDA graphs) so that
      every kernel shows in a launch list:
        ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file out.csv python scripts/profile_layered.py steps ...
  python scripts/profile_layered.py window-attention
      the windowed-attention tile kernel alone (2048 rows of one sequence, 16 / 8 heads of 128, 64 rotated dims, window
      1024, soft cap 50), timed with CUDA events; small enough for a full counter capture:
        ncu --set full --clock-control none -k regex:window_attention_mma -s 1 -c 2 -o out python scripts/profile_layered.py window-attention
  python scripts/profile_layered.py lightning-scan
      the chunk-parallel linear-attention scan alone (2048 rows of one sequence, 16 heads of 128 x 128), timed with CUDA
      events, then the token-by-token kernel on 32 sequences of one row:
        ncu --set full --clock-control none -k regex:lightning_chunk_out -s 1 -c 2 -o out python scripts/profile_layered.py lightning-scan
  python scripts/profile_layered.py talk-attention
      the head-mixed attention tile kernel alone (2048 rows of one sequence, 16 / 4 heads, keys and values of 128, 64
      rotated dims, the head mix folded into queries of 4 x 128), timed with CUDA events:
        ncu --set full --clock-control none -k regex:talk_attention_mma -s 1 -c 1 -o out python scripts/profile_layered.py talk-attention
Run the plain command first; capture only if it exits 0.
"""
import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def steps(a):
    os.environ["DLLAMA_LAYERS_GRAPHS"] = "0"
    import numpy as np
    import torch
    import bench
    from dllama_b200.models import registry
    from dllama_b200.models.layered import write_random_model
    T, users, vocab, nl = a.prompt, 32, 32768, a.layers
    d = os.path.join(a.model_dir, f"dllama_b200_{'layered' if a.design == 'ribivik' else a.design}_{a.size}_l{nl}")
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        cfg = {"ribivik": lambda: bench.layered_config(bench.LAYERED_SIZES[a.size], nl, vocab), "sunesun": lambda: bench.sunesun_config(a.size, nl, vocab),
               "venadra": lambda: bench.venadra_config(a.size, nl, vocab), "darusun": lambda: bench.darusun_config(a.size, nl, vocab)}[a.design]()
        write_random_model(d, cfg, seed=1)
    torch.cuda.set_device(0)
    eng = registry.engine_for_dir(d, max_rows=T, n_slots=users, max_seq_len=T + 64, dtype="bfloat16")
    prompt = np.random.default_rng(0).integers(1, vocab, T).tolist()
    slots = [eng.alloc_slot() for _ in range(users)]
    for s in slots:
        eng.forward(prompt, list(range(T)), [s] * T, logits_from=T - 1)
    torch.cuda.synchronize()
    print("prompts done: %d forwards of %d rows" % (users, T))
    for i in range(3):
        eng.decode_step_greedy([1], [T + i], [slots[0]])
    torch.cuda.synchronize()
    print("3 decode steps of 1 row done")
    for i in range(2):
        eng.decode_step_greedy([1] * users, [T + 3 + i] + [T + i] * (users - 1), slots)
    torch.cuda.synchronize()
    print("2 decode steps of %d rows done" % users)


def window_attention(a):
    import torch
    from dllama_b200.models.layered import interpolated_rotary
    from dllama_b200.ops import layers as L
    H, G, d, rd, window, cap, n = 16, 8, 128, 64, 1024, 50.0, 2048
    f, mag = interpolated_rotary(10000.0, rd, None)
    n_pages = n // 32
    bt = torch.arange(n_pages, dtype=torch.int32).view(1, -1).cuda()
    cache = torch.zeros(n_pages, G, 32, d + rd, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator().manual_seed(1)
    k, q = torch.randn(n, G * d, generator=g).cuda(), torch.randn(n, H * d, generator=g).cuda()
    pos, slot = torch.arange(n, dtype=torch.int32).cuda(), torch.zeros(n, dtype=torch.int32).cuda()
    L.window_kv_write(k, n, G, d, rd, f.cuda(), mag, pos, slot, bt, cache, q=q, q_heads=H)
    out = torch.zeros(n, H * d, device="cuda")
    rq = L.window_tc_rows(H, G)
    tiles = torch.arange(n, dtype=torch.int32).view(-1, rq).cuda()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(4):
        ev0.record()
        L.window_attention_tc(q, out, H, G, d, rd, 1 / math.sqrt(d), cap, window, pos, slot, bt, cache, tiles, n // rq, rq)
        ev1.record()
        torch.cuda.synchronize()
        print("window attention: %.1f us" % (ev0.elapsed_time(ev1) * 1e3))
    keys = sum(min(i + 1, window) for i in range(n))
    print("GFLOP over the visible keys: %.2f" % (keys * H * d * 4 / 1e9))


def talk_attention(a):
    import torch
    from dllama_b200.models.layered import rotary_frequencies
    from dllama_b200.ops import layers as L
    H, G, d, dv, rd, n = 16, 4, 128, 128, 64, 2048
    n_pages = n // 32
    bt = torch.arange(n_pages, dtype=torch.int32).view(1, -1).cuda()
    cache = torch.zeros(n_pages, G, 32, d + dv, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(n, w, generator=g).cuda() for w in (H * d, G * d, G * dv))
    talk = (torch.eye(H) + torch.randn(H, H, generator=g) * 0.3).cuda()
    qm = torch.zeros(n, H * G * d, device="cuda")
    pos, slot = torch.arange(n, dtype=torch.int32).cuda(), torch.zeros(n, dtype=torch.int32).cuda()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    freqs = rotary_frequencies(500000.0, rd).cuda()
    for _ in range(3):
        ev0.record()
        L.window_kv_write(k, n, G, d, rd, freqs, 1.0, pos, slot, bt, cache, q=q, q_heads=H, v=v, vdim=dv,
                          qk_norm=True, eps=1e-5, rope_half=True, talk=talk, q_mixed=qm)
        ev1.record()
        torch.cuda.synchronize()
        print("cache writer (rotary, unit norms, head mix): %.1f us" % (ev0.elapsed_time(ev1) * 1e3))
    out = torch.zeros(n, H * dv, device="cuda")
    rq = L.talk_tc_rows(H, G, d, dv, G, n)
    tiles = torch.arange(n, dtype=torch.int32).view(-1, rq).cuda()
    for n_splits in (1, 4):
        part = torch.zeros(L.talk_tc_partial_floats(n // rq, G, n_splits, dv, rq, H), device="cuda") if n_splits > 1 else None
        for _ in range(4):
            ev0.record()
            L.talk_attention_tc(qm, out, H, G, d, dv, 0.1, 0, pos, slot, bt, cache, tiles, n // rq, rq, n_splits, part, key_heads=G)
            ev1.record()
            torch.cuda.synchronize()
            print("head-mixed attention, tiles of %d rows, %d page shares: %.1f us" % (rq, n_splits, ev0.elapsed_time(ev1) * 1e3))
    pairs = n * (n + 1) // 2
    print("FLOPs per launch (visible pairs, folded form 2 * (4 * 128 + 128) per head): %.1f G" % (pairs * H * 2 * (G * d + dv) / 1e9))


def lightning_scan(a):
    import torch
    from dllama_b200.ops import layers as L
    H, d, dv, n, users = 16, 128, 128, 2048, 32
    g = torch.Generator().manual_seed(1)
    qkv = (torch.randn(n, H * (2 * d + dv), generator=g) * 0.3).cuda()
    decay = torch.linspace(0.6, 0.999, H).cuda()
    y = torch.zeros(n, H * dv, device="cuda")
    state = torch.zeros(users, H, d, dv, device="cuda")
    scratch = torch.zeros(L.lightning_chunk_floats(n, 1, H, d, dv), device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    keep = [i32(list(range(n))), i32([0] * n), i32([0, n]), i32(list(range(n))), i32([0]), i32([0])]
    b = L.mamba_batch(*keep)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(4):
        ev0.record()
        L.lightning_scan(b, 1, qkv, qkv[:, H * d:], qkv[:, 2 * H * d:], decay, y, state, H, d, dv, max_chunks=n // L.LIGHTNING_CHUNK, scratch=scratch)
        ev1.record()
        torch.cuda.synchronize()
        print("chunked scan, %d rows: %.1f us" % (n, ev0.elapsed_time(ev1) * 1e3))
    print("GFLOP (state update and read-out, 4 dim vdim per row and head): %.2f" % (n * H * 4 * d * dv / 1e9))
    keep2 = [i32([5] * users), i32(list(range(users))), i32(list(range(users + 1))), i32(list(range(users))), i32(list(range(users))), i32([5] * users)]
    b2 = L.mamba_batch(*keep2)
    for m in (1, users):
        for _ in range(3):
            ev0.record()
            L.lightning_scan(b2, m, qkv, qkv[:, H * d:], qkv[:, 2 * H * d:], decay, y, state, H, d, dv)
            ev1.record()
            torch.cuda.synchronize()
            print("token-by-token scan, %d sequences of one row: %.1f us for %.1f MB of state read and written" % (m, ev0.elapsed_time(ev1) * 1e3, 2 * m * H * d * dv * 4 / 1e6))


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=("steps", "window-attention", "lightning-scan", "talk-attention"))
    ap.add_argument("--design", default="sunesun", choices=("ribivik", "sunesun", "venadra", "darusun"))
    ap.add_argument("--size", default="w2048")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--model-dir", default="/tmp")
    a = ap.parse_args()
    {"steps": steps, "window-attention": window_attention, "lightning-scan": lightning_scan, "talk-attention": talk_attention}[a.what](a)
