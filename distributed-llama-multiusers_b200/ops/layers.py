"""Torch-tensor wrappers over the layer-list model kernels (libdllama_b200_layers.so; C ABI in include/dllama_b200.h).

One function per kernel launch, all on ``torch.cuda.current_stream()``; nothing here allocates.  Activations are f32
tensors; weights are bf16 or f32 tensors (``wtype`` follows the tensor's dtype), caches likewise.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib
from .lib import (DENSE_GLU_CLAMP, DENSE_GLU_SILU, DENSE_MUL, DENSE_RELU2, DENSE_ROWGATE_ADD, DENSE_SIGMOID_MUL, DENSE_SILU, DENSE_SOFTCAP, DENSE_STORE,  # noqa: F401
                  DENSE_XIELU, EPI_DENSE, T_BF16, T_F32,
                  DlConvArgs, DlDenseArgs, DlEpilogue, DlHyperArgs, DlLatentAttnArgs, DlLightningArgs, DlLatentKvArgs, DlLatentTiles, DlMambaBatch, DlMambaChunks, DlMambaScanArgs, DlMoeArgs,
                  DlMoePlanArgs, DlMoeSelectArgs, DlNormArgs, DlWindowAttnArgs, DlWindowKvArgs, check_layers, layers_lib)

PAGE_SIZE = 32
HC_MAX_STREAMS = 16          # DL_HC_MAX_STREAMS of the hyper-connection kernel


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _type(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return T_BF16
    if t.dtype == torch.float32:
        return T_F32
    raise TypeError(f"layer kernels take bf16 or f32 weights and caches, not {t.dtype}")


def sm_count() -> int:
    return int(layers_lib().dl_device_sm_count())


def embed_rows(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, M: int, scale: float = 1.0, copies: int = 1):
    """x[m][c] = scale * table[tokens[m]] for each of `copies` copies of a row (x rows are [copies][dim])."""
    check_layers(layers_lib().dl_embed_rows(table.data_ptr(), _type(table), tokens.data_ptr(), x.data_ptr(), M,
                                            table.shape[1], scale, copies, _stream()), "dl_embed_rows")
    lib.count_launch()


def dense(w: torch.Tensor, x: torch.Tensor, y: torch.Tensor, M: int, round_x: bool, epi: int = DENSE_STORE,
          aux: Optional[torch.Tensor] = None, param: float = 0.0, param2: float = 0.0):
    """y[:M] = epi(x[:M] @ w^T); w [N][K] (rows may be strided), x [.., >= K] and y [.., >= N] row-major f32."""
    N, K = w.shape
    a = DlDenseArgs()
    a.W, a.wtype, a.ldw, a.w_bs = w.data_ptr(), _type(w), w.stride(0), 0
    a.X, a.ldx, a.x_bs = x.data_ptr(), x.stride(0), 0
    a.Y, a.ldy, a.y_bs = y.data_ptr(), y.stride(0), 0
    a.M, a.N, a.K, a.batch = M, N, K, 1
    a.round_x, a.epi = 1 if round_x else 0, epi
    a.aux, a.ld_aux, a.aux_bs = _p(aux), (aux.stride(0) if aux is not None else 0), 0
    a.param, a.param2 = param, param2
    check_layers(layers_lib().dl_dense(a, _stream()), "dl_dense")
    lib.count_launch()


def dense_heads(w: torch.Tensor, x: torch.Tensor, y: torch.Tensor, M: int, round_x: bool, x_head_stride: int,
                y_head_stride: int):
    """Per-head products in one launch: y[m, h*ys : h*ys + N] = x[m, h*xs : h*xs + K] @ w[h]^T for w [H][N][K]."""
    H, N, K = w.shape
    a = DlDenseArgs()
    a.W, a.wtype, a.ldw, a.w_bs = w.data_ptr(), _type(w), w.stride(1), w.stride(0)
    a.X, a.ldx, a.x_bs = x.data_ptr(), x.stride(0), x_head_stride
    a.Y, a.ldy, a.y_bs = y.data_ptr(), y.stride(0), y_head_stride
    a.M, a.N, a.K, a.batch = M, N, K, H
    a.round_x, a.epi = 1 if round_x else 0, DENSE_STORE
    a.aux, a.ld_aux, a.aux_bs, a.param, a.param2 = None, 0, 0, 0.0, 0.0
    check_layers(layers_lib().dl_dense(a, _stream()), "dl_dense")
    lib.count_launch()


# ---- tensor-core path (bf16 weights, many rows): the tcgen05 GEMM of gemm_wh_tc.cu on pre-tiled operand images -----
def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def make_wh(w: torch.Tensor) -> torch.Tensor:
    """bf16 [N][K] (rows may be strided) -> the weight image of the tcgen05 GEMM (allocates; zero-padded to 128 x 128 tiles)."""
    assert w.dtype == torch.bfloat16 and w.stride(1) == 1
    N, K = w.shape
    out = torch.empty(int(layers_lib().dl_wh_bytes(N, _round_up(K, 128))), dtype=torch.uint8, device=w.device)
    check_layers(layers_lib().dl_wh_from_dense(w.data_ptr(), N, K, w.stride(0), out.data_ptr(), _stream()), "dl_wh_from_dense")
    lib.count_launch()
    return out


def xh_bytes(K: int, ncap: int) -> int:
    return _round_up(K, 128) // 128 * (ncap // 8) * 2048


def xh_from_rows(x: torch.Tensor, M: int, K: int, ncap: int, xh: torch.Tensor):
    """Columns [0, K) of the first M rows of f32 x -> bf16 activation slabs of the tcgen05 GEMM."""
    assert xh.numel() >= xh_bytes(K, ncap)
    check_layers(layers_lib().dl_xh_from_rows(x.data_ptr(), x.stride(0), M, K, ncap, xh.data_ptr(), _stream()), "dl_xh_from_rows")
    lib.count_launch()


def dense_tc(wh: torch.Tensor, N: int, K: int, xh: torch.Tensor, ncap: int, y: torch.Tensor, M: int, epi: int = DENSE_STORE,
             aux: Optional[torch.Tensor] = None, param: float = 0.0, param2: float = 0.0):
    """y[:M, :N] = epi(x @ w^T) from the two operand images (bf16 x bf16 -> f32 in tensor memory)."""
    e = DlEpilogue()
    e.kind, e.n_dst, e.ld, e.dst_off = EPI_DENSE, 1, y.stride(0), 0
    e.dst[0] = y.data_ptr()
    e.dense_op, e.dense_param, e.dense_param2 = epi, param, param2
    e.dense_aux, e.dense_aux_ld = _p(aux), (aux.stride(0) if aux is not None else 0)
    check_layers(layers_lib().dl_gemm_wh_tc(wh.data_ptr(), N, _round_up(K, 128), xh.data_ptr(), ncap, M, e, 2, 0, _stream()),
                 "dl_gemm_wh_tc")
    lib.count_launch()


def rms_norm(x: torch.Tensor, y: torch.Tensor, M: int, dim: int, eps: float, w: Optional[torch.Tensor] = None,
             plus_one: bool = False, groups: int = 1, gate: Optional[torch.Tensor] = None, accumulate: bool = False,
             rows: Optional[torch.Tensor] = None):
    a = DlNormArgs()
    a.x, a.ldx = x.data_ptr(), x.stride(0)
    a.gate, a.ld_gate = _p(gate), (gate.stride(0) if gate is not None else 0)
    a.w, a.y, a.ldy, a.rows = _p(w), y.data_ptr(), y.stride(0), _p(rows)
    a.M, a.dim, a.groups, a.eps = M, dim, groups, eps
    a.plus_one, a.accumulate = 1 if plus_one else 0, 1 if accumulate else 0
    check_layers(layers_lib().dl_rms_norm(a, _stream()), "dl_rms_norm")
    lib.count_launch()


def poly_norm(x: torch.Tensor, y: torch.Tensor, M: int, dim: int, coef: torch.Tensor, eps: float):
    """y = c0 N(x) + c1 N(x^2) + c2 N(x^3) + c3 per row, N(u) = u / sqrt(mean(u^2) + eps); coef: 4 f32 on the device."""
    assert coef.dtype == torch.float32 and coef.numel() == 4
    check_layers(layers_lib().dl_poly_norm(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), M, dim, coef.data_ptr(), eps, _stream()),
                 "dl_poly_norm")
    lib.count_launch()


def latent_kv_write(kv: torch.Tensor, M: int, norm_w: torch.Tensor, eps: float, rank: int, rot: int, rope_dims: int,
                    freqs: torch.Tensor, pos, slot, block_table: torch.Tensor, cache: torch.Tensor, interleaved: bool = False):
    a = DlLatentKvArgs()
    a.interleaved = 1 if interleaved else 0
    a.kv, a.ld, a.norm_w, a.eps = kv.data_ptr(), kv.stride(0), norm_w.data_ptr(), eps
    a.rank, a.rot, a.rope_dims, a.freqs = rank, rot, rope_dims, freqs.data_ptr()
    a.pos, a.slot, a.block_table = pos.data_ptr(), slot.data_ptr(), block_table.data_ptr()
    a.max_pages, a.page_size = block_table.shape[1], PAGE_SIZE
    a.cache, a.ctype = cache.data_ptr(), _type(cache)
    check_layers(layers_lib().dl_latent_kv_write(a, M, _stream()), "dl_latent_kv_write")
    lib.count_launch()


def rope_rows(x: torch.Tensor, M: int, n_heads: int, head_stride: int, offset: int, rope_dims: int, freqs: torch.Tensor,
              pos: torch.Tensor, interleaved: bool = False, mag: float = 1.0):
    """Rotary on dims [offset, offset + rope_dims) of every head, in place; pairs (i, i + dims/2) or, interleaved,
    (2i, 2i + 1); cos and sin are multiplied by `mag`."""
    check_layers(layers_lib().dl_rope_rows(x.data_ptr(), x.stride(0), M, n_heads, head_stride, offset, rope_dims,
                                           freqs.data_ptr(), pos.data_ptr(), 1 if interleaved else 0, mag, _stream()), "dl_rope_rows")
    lib.count_launch()


LATENT_TC_ROWS = 64          # most stacked (query row x head) rows of one tile of the tensor-core kernel


def latent_tc_supported(n_heads: int, rank: int, rot: int, cache_dtype, rq: int) -> bool:
    ctype = T_BF16 if cache_dtype == torch.bfloat16 else T_F32
    return layers_lib().dl_latent_attention_tc_supported(n_heads, rank, rot, ctype, rq) == 0


def latent_tc_partial_floats(n_tiles: int, n_splits: int, rank: int) -> int:
    return int(layers_lib().dl_latent_tc_partial_floats(n_tiles, n_splits, rank))


def latent_attention(q_lat: torch.Tensor, q: torch.Tensor, q_head_stride: int, q_rot_offset: int, out: torch.Tensor,
                     M: int, n_heads: int, rank: int, rot: int, scale: float, pos, slot, block_table: torch.Tensor,
                     cache: torch.Tensor, tiles=None, window: int = 0, sink: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None):
    """tiles = (tile_rows int32 [n_tiles][rq], n_tiles, rq, n_splits, partial f32 or None): the tensor-core kernel over
    row tiles of one sequence each (bf16 cache); None: the per-row kernel (any cache type).  window > 0: a position sees
    itself and the window - 1 before it; sink [heads]: joins the softmax denominator; gate [M][>= heads]: head h of row m
    leaves multiplied by sigmoid(gate[m][h])."""
    a = DlLatentAttnArgs()
    a.q_lat, a.q, a.ldq = q_lat.data_ptr(), q.data_ptr(), q.stride(0)
    a.q_head_stride, a.q_rot_offset, a.out = q_head_stride, q_rot_offset, out.data_ptr()
    a.n_heads, a.rank, a.rot, a.scale = n_heads, rank, rot, scale
    a.pos, a.slot, a.block_table = pos.data_ptr(), slot.data_ptr(), block_table.data_ptr()
    a.max_pages, a.page_size = block_table.shape[1], PAGE_SIZE
    a.cache, a.ctype = cache.data_ptr(), _type(cache)
    a.window, a.sink, a.gate, a.ld_gate = window, _p(sink), _p(gate), (gate.stride(0) if gate is not None else 0)
    if tiles is not None:
        t = DlLatentTiles()
        t.tile_rows, t.n_tiles, t.rq, t.n_splits, t.partial = tiles[0].data_ptr(), tiles[1], tiles[2], tiles[3], _p(tiles[4])
        check_layers(layers_lib().dl_latent_attention_tc(a, t, _stream()), "dl_latent_attention_tc")
        lib.count_launch(2 if tiles[3] > 1 else 1)
        return
    check_layers(layers_lib().dl_latent_attention(a, M, _stream()), "dl_latent_attention")
    lib.count_launch()


def mamba_batch(pos, row_seq, seq_start, seq_rows, seq_slot, seq_pos0) -> DlMambaBatch:
    b = DlMambaBatch()
    b.pos, b.row_seq, b.seq_start = pos.data_ptr(), row_seq.data_ptr(), seq_start.data_ptr()
    b.seq_rows, b.seq_slot, b.seq_pos0 = seq_rows.data_ptr(), seq_slot.data_ptr(), seq_pos0.data_ptr()
    return b


def mamba_conv(batch: DlMambaBatch, M: int, n_seq: int, zx: torch.Tensor, in_off: int, w: torch.Tensor,
               bias: torch.Tensor, conv_state: torch.Tensor, out: torch.Tensor):
    channels, taps = w.shape
    assert bias.dtype == w.dtype and out.stride(0) == channels
    check_layers(layers_lib().dl_mamba_conv(batch, M, n_seq, zx.data_ptr(), zx.stride(0), in_off, w.data_ptr(),
                                            bias.data_ptr(), _type(w), conv_state.data_ptr(), out.data_ptr(), channels,
                                            taps, _stream()), "dl_mamba_conv")
    lib.count_launch(2 if taps > 1 else 1)


def causal_conv(batch: DlMambaBatch, M: int, n_seq: int, x: torch.Tensor, w: torch.Tensor, conv_state: torch.Tensor,
                out: torch.Tensor, bias: Optional[torch.Tensor] = None, act: bool = False, residual: bool = False, in_off: int = 0):
    """out[m][ch] = act(bias + sum_k w[ch][k] x[position - (taps - 1) + k][ch]) (+ x[m][ch]); zeros before a sequence's
    start; conv_state [slots][taps - 1][channels] carries every slot's last inputs and is updated."""
    channels, taps = w.shape
    a = DlConvArgs()
    a.in_, a.ld, a.in_off = x.data_ptr(), x.stride(0), in_off
    a.w, a.bias, a.wtype, a.conv_state = w.data_ptr(), _p(bias), _type(w), conv_state.data_ptr()
    a.out, a.ld_out = out.data_ptr(), out.stride(0)
    a.channels, a.taps, a.act, a.residual = channels, taps, 1 if act else 0, 1 if residual else 0
    check_layers(layers_lib().dl_causal_conv(batch, M, n_seq, a, _stream()), "dl_causal_conv")
    lib.count_launch(2 if taps > 1 else 1)


LIGHTNING_CHUNK = 64         # DL_LIGHTNING_CHUNK: rows of a sequence per chunk of the chunked linear-attention scan


def lightning_chunked_supported(dim: int, vdim: int) -> bool:
    return layers_lib().dl_lightning_scan_chunked_supported(dim, vdim) == 0


def lightning_chunk_floats(M: int, n_seq: int, n_heads: int, dim: int, vdim: int) -> int:
    return int(layers_lib().dl_lightning_chunk_floats(M, n_seq, n_heads, dim, vdim))


def lightning_scan(batch: DlMambaBatch, n_seq: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                   y: torch.Tensor, state: torch.Tensor, n_heads: int, dim: int, vdim: int, max_chunks: int = 0,
                   scratch: Optional[torch.Tensor] = None):
    """Linear attention with a decay per head: S <- decay S + k v^T, y = S^T q per row, state [slots][heads][dim][vdim] f32.
    max_chunks > 0 (with scratch): the chunk-parallel form for long portions."""
    a = DlLightningArgs()
    a.q, a.k, a.v, a.ldq, a.ldk, a.ldv = q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0)
    a.decay, a.y, a.ld_y, a.state = decay.data_ptr(), y.data_ptr(), y.stride(0), state.data_ptr()
    a.n_heads, a.dim, a.vdim = n_heads, dim, vdim
    if max_chunks > 0:
        check_layers(layers_lib().dl_lightning_scan_chunked(batch, n_seq, max_chunks, a, scratch.data_ptr(), _stream()),
                     "dl_lightning_scan_chunked")
        lib.count_launch(3)
        return
    check_layers(layers_lib().dl_lightning_scan(batch, n_seq, a, _stream()), "dl_lightning_scan")
    lib.count_launch()


MAMBA_CHUNK = 128            # rows of a sequence per chunk of the chunked scan


def mamba_chunked_supported(vdim: int, state: int) -> bool:
    return layers_lib().dl_mamba_scan_chunked_supported(vdim, state) == 0


def mamba_scan(batch: DlMambaBatch, n_seq: int, xbc: torch.Tensor, dt: torch.Tensor, dt_bias, A_log, D, y: torch.Tensor,
               ssm_state: torch.Tensor, n_heads: int, vdim: int, state: int, groups: int, chunks=None):
    """dt: a view whose element [m, h] is the raw step size of head h of row m.  chunks = (chunk_seq, chunk_off, n_chunks,
    state scratch, decay scratch, cum scratch): the two-pass scan over chunks of MAMBA_CHUNK rows run in parallel."""
    a = DlMambaScanArgs()
    a.xbc, a.ld_xbc, a.dt, a.ld_dt = xbc.data_ptr(), xbc.stride(0), dt.data_ptr(), dt.stride(0)
    a.dt_bias, a.A_log, a.D = dt_bias.data_ptr(), A_log.data_ptr(), D.data_ptr()
    a.y, a.ld_y, a.ssm_state = y.data_ptr(), y.stride(0), ssm_state.data_ptr()
    a.n_heads, a.vdim, a.state, a.groups = n_heads, vdim, state, groups
    if chunks is not None:
        c = DlMambaChunks()
        c.chunk_seq, c.chunk_off, c.n_chunks, c.chunk = chunks[0].data_ptr(), chunks[1].data_ptr(), chunks[2], MAMBA_CHUNK
        c.state, c.decay, c.cum = chunks[3].data_ptr(), chunks[4].data_ptr(), chunks[5].data_ptr()
        check_layers(layers_lib().dl_mamba_scan_chunked(batch, a, c, _stream()), "dl_mamba_scan_chunked")
        lib.count_launch(2)
        return
    check_layers(layers_lib().dl_mamba_scan(batch, n_seq, a, _stream()), "dl_mamba_scan")
    lib.count_launch()


# ---- hyper-connections ------------------------------------------------------------------------------------------------
def hyper_step(x: torch.Tensor, M: int, streams: int, dim: int, y: Optional[torch.Tensor] = None,
               mix: Optional[torch.Tensor] = None, w_out: Optional[torch.Tensor] = None, mult: float = 1.0,
               h: Optional[torch.Tensor] = None, w_in: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
               eps: float = 0.0, rows: Optional[torch.Tensor] = None, u_out: Optional[torch.Tensor] = None):
    """x [rows][streams * dim] f32.  With y: every copy is rewritten from the old ones (mix [from][to]) plus
    mult * w_out[t] * y.  With h: h = rms_norm(sum_s w_in[s] x_s) * norm_w of the (new) copies.  One launch."""
    a = DlHyperArgs()
    a.x, a.ldx, a.streams, a.dim, a.M = x.data_ptr(), x.stride(0), streams, dim, M
    a.y, a.ldy = _p(y), (y.stride(0) if y is not None else 0)
    a.mix, a.w_out, a.mult = _p(mix), _p(w_out), mult
    a.w_in, a.norm_w, a.eps, a.rows = _p(w_in), _p(norm_w), eps, _p(rows)
    a.h, a.ldh, a.u_out = _p(h), (h.stride(0) if h is not None else 0), _p(u_out)
    check_layers(layers_lib().dl_hyper_step(a, _stream()), "dl_hyper_step")
    lib.count_launch()


# ---- sliding-window attention whose values are its keys ---------------------------------------------------------------
def window_kv_write(k: Optional[torch.Tensor], M: int, kv_heads: int, dim: int, rope_dims: int, freqs: torch.Tensor, rope_scale: float,
                    pos, slot, block_table: torch.Tensor, cache: torch.Tensor, q: Optional[torch.Tensor] = None, q_heads: int = 0,
                    v: Optional[torch.Tensor] = None, vdim: int = 0, qk_norm: bool = False, eps: float = 0.0, rope_half: bool = False,
                    talk: Optional[torch.Tensor] = None, q_mixed: Optional[torch.Tensor] = None):
    """Keys into the paged cache (rotated key + unrotated head per line); with q [M][q_heads * dim] the queries are
    rotated in place by the same launch.  With v [M][kv_heads * vdim] the line is key + value; rotary (pairs (i, i + dims / 2)
    with rope_half, else (2i, 2i + 1)) comes first, then qk_norm divides every query and key head by its root mean square.
    talk [q_heads][q_heads] f32 with q_mixed [M][q_heads * kv_heads * dim]: the head mix of the scores, folded into the queries."""
    a = DlWindowKvArgs()
    a.k, a.ld, a.kv_heads, a.dim, a.rope_dims = _p(k), (k.stride(0) if k is not None else 0), kv_heads, dim, rope_dims
    a.q, a.ldq, a.q_heads = _p(q), (q.stride(0) if q is not None else 0), q_heads
    a.freqs, a.rope_scale = freqs.data_ptr(), rope_scale
    a.pos, a.slot, a.block_table = pos.data_ptr(), slot.data_ptr(), block_table.data_ptr()
    a.max_pages, a.page_size = block_table.shape[1], PAGE_SIZE
    a.cache, a.ctype = cache.data_ptr(), _type(cache)
    a.v, a.ldv, a.vdim = _p(v), (v.stride(0) if v is not None else 0), vdim
    a.qk_norm, a.eps = 1 if qk_norm else 0, eps
    a.rope_half, a.talk, a.q_mixed, a.ld_qm = 1 if rope_half else 0, _p(talk), _p(q_mixed), (q_mixed.stride(0) if q_mixed is not None else 0)
    check_layers(layers_lib().dl_window_kv_write(a, M, _stream()), "dl_window_kv_write")
    lib.count_launch()


def _window_args(q, out, heads, kv_heads, dim, rope_dims, scale, softcap, window, pos, slot, block_table, cache,
                 vdim: int = 0, chunk: int = 0, sink: Optional[torch.Tensor] = None, key_heads: int = 0):
    a = DlWindowAttnArgs()
    a.q, a.ldq, a.out, a.ldo = q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)
    a.heads, a.kv_heads, a.dim, a.rope_dims = heads, kv_heads, dim, rope_dims
    a.scale, a.softcap, a.window = scale, softcap, window
    a.pos, a.slot, a.block_table = pos.data_ptr(), slot.data_ptr(), block_table.data_ptr()
    a.max_pages, a.page_size = block_table.shape[1], PAGE_SIZE
    a.cache, a.ctype = cache.data_ptr(), _type(cache)
    a.vdim, a.chunk, a.sink, a.key_heads = vdim, chunk, _p(sink), key_heads
    return a


def window_attention(q: torch.Tensor, out: torch.Tensor, M: int, heads: int, kv_heads: int, dim: int, rope_dims: int,
                     scale: float, softcap: float, window: int, pos, slot, block_table: torch.Tensor, cache: torch.Tensor,
                     vdim: int = 0, chunk: int = 0, sink: Optional[torch.Tensor] = None, key_heads: int = 0):
    """The per-row kernel (either cache type, f32 arithmetic).  vdim > 0: values of their own behind the keys; chunk > 0:
    only keys of the row's own chunk of positions are visible; sink [heads]: joins the softmax denominator; key_heads =
    kv_heads: q is [M][heads][kv_heads * dim] (head-mixed queries) against the keys of all key/value heads side by side."""
    a = _window_args(q, out, heads, kv_heads, dim, rope_dims, scale, softcap, window, pos, slot, block_table, cache, vdim, chunk, sink, key_heads)
    check_layers(layers_lib().dl_window_attention(a, M, _stream()), "dl_window_attention")
    lib.count_launch()


def window_tc_rows(heads: int, kv_heads: int) -> int:
    """Rows of one sequence per tile of the tensor-core kernel (0: more heads per group than it stacks)."""
    return int(layers_lib().dl_window_tc_rows(heads, kv_heads))


def window_tc_supported(heads: int, kv_heads: int, dim: int, rope_dims: int, cache_dtype) -> bool:
    ctype = T_BF16 if cache_dtype == torch.bfloat16 else T_F32
    return layers_lib().dl_window_attention_tc_supported(heads, kv_heads, dim, rope_dims, ctype) == 0


def window_tc_partial_floats(n_tiles: int, kv_heads: int, n_splits: int, dim: int) -> int:
    return int(layers_lib().dl_window_tc_partial_floats(n_tiles, kv_heads, n_splits, dim))


def window_attention_tc(q: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dim: int, rope_dims: int, scale: float,
                        softcap: float, window: int, pos, slot, block_table: torch.Tensor, cache: torch.Tensor,
                        tile_rows: torch.Tensor, n_tiles: int, rq: int, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                        vdim: int = 0, chunk: int = 0, sink: Optional[torch.Tensor] = None):
    """The tensor-core kernel over row tiles (tile_rows int32 [n_tiles][rq] on the device, -1 = no row).  n_splits > 1:
    that many CTAs share each tile's pages (few tiles: decoding) and a merge launch follows; partial: f32 scratch."""
    a = _window_args(q, out, heads, kv_heads, dim, rope_dims, scale, softcap, window, pos, slot, block_table, cache, vdim, chunk, sink)
    if n_splits > 1:
        assert partial is not None and partial.numel() >= window_tc_partial_floats(n_tiles, kv_heads, n_splits, dim)
    check_layers(layers_lib().dl_window_attention_tc(a, tile_rows.data_ptr(), n_tiles, rq, n_splits, _p(partial), _stream()),
                 "dl_window_attention_tc")
    lib.count_launch(2 if n_splits > 1 else 1)


def talk_tc_supported(heads: int, kv_heads: int, dim: int, vdim: int, key_heads: int, cache_dtype) -> bool:
    ctype = T_BF16 if cache_dtype == torch.bfloat16 else T_F32
    return layers_lib().dl_talk_attention_tc_supported(heads, kv_heads, dim, vdim, key_heads, ctype) == 0


def talk_tc_rows(heads: int, kv_heads: int, dim: int, vdim: int, key_heads: int, longest: int) -> int:
    """Rows of one sequence per tile of the kernel for portions of up to `longest` rows: the tile stacks 16 (decoding), 64
    or 128 (row, head-of-a-group) pairs, whichever fits the shared memory."""
    return int(layers_lib().dl_talk_tc_tile_rows(heads, kv_heads, dim, vdim, key_heads, longest)) // (heads // kv_heads)


def talk_tc_partial_floats(n_tiles: int, kv_heads: int, n_splits: int, vdim: int, rq: int, heads: int) -> int:
    stacked = rq * (heads // kv_heads)
    return int(layers_lib().dl_talk_tc_partial_floats(n_tiles, kv_heads, n_splits, vdim, 16 if stacked <= 16 else 64 if stacked <= 64 else 128))


def talk_attention_tc(q: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, window: int,
                      pos, slot, block_table: torch.Tensor, cache: torch.Tensor, tile_rows: torch.Tensor, n_tiles: int, rq: int,
                      n_splits: int = 1, partial: Optional[torch.Tensor] = None, chunk: int = 0, sink: Optional[torch.Tensor] = None,
                      key_heads: int = 0):
    """The tile kernel for values of their own width and (key_heads = kv_heads) head-mixed queries [M][heads][kv_heads * dim]
    against the keys of all key/value heads side by side.  Tiles and page shares as in window_attention_tc."""
    a = _window_args(q, out, heads, kv_heads, dim, 0, scale, 0.0, window, pos, slot, block_table, cache, vdim, chunk, sink, key_heads)
    if n_splits > 1:
        assert partial is not None and partial.numel() >= talk_tc_partial_floats(n_tiles, kv_heads, n_splits, vdim, rq, heads)
    check_layers(layers_lib().dl_talk_attention_tc(a, tile_rows.data_ptr(), n_tiles, rq, n_splits, _p(partial), _stream()),
                 "dl_talk_attention_tc")
    lib.count_launch(2 if n_splits > 1 else 1)


def talk_attention_tiles(q, out, heads, kv_heads, dim, vdim, scale, window, pos, slot, block_table, cache, tiles, rq: int, n_splits: int = 1,
                         chunk: int = 0, sink: Optional[torch.Tensor] = None, key_heads: int = 0):
    """Convenience for callers with host-side tiles (lists of up to rq row indices of one sequence, consecutive positions)."""
    t = torch.full((len(tiles), rq), -1, dtype=torch.int32)
    for i, rows in enumerate(tiles):
        t[i, :len(rows)] = torch.tensor(rows, dtype=torch.int32)
    partial = None
    if n_splits > 1:
        partial = torch.zeros(talk_tc_partial_floats(len(tiles), kv_heads, n_splits, vdim, rq, heads), dtype=torch.float32, device=q.device)
    talk_attention_tc(q, out, heads, kv_heads, dim, vdim, scale, window, pos, slot, block_table, cache, t.to(q.device), len(tiles), rq,
                      n_splits, partial, chunk, sink, key_heads)


def window_attention_tiles(q, out, heads, kv_heads, dim, rope_dims, scale, softcap, window, pos, slot, block_table, cache, tiles,
                           n_splits: int = 1, vdim: int = 0, chunk: int = 0, sink: Optional[torch.Tensor] = None):
    """Convenience for callers with host-side tiles (lists of row indices of one sequence, consecutive positions)."""
    rq = window_tc_rows(heads, kv_heads)
    t = torch.full((len(tiles), rq), -1, dtype=torch.int32)
    for i, rows in enumerate(tiles):
        t[i, :len(rows)] = torch.tensor(rows, dtype=torch.int32)
    partial = None
    if n_splits > 1:
        partial = torch.zeros(window_tc_partial_floats(len(tiles), kv_heads, n_splits, dim), dtype=torch.float32, device=q.device)
    window_attention_tc(q, out, heads, kv_heads, dim, rope_dims, scale, softcap, window, pos, slot, block_table, cache,
                        t.to(q.device), len(tiles), rq, n_splits, partial, vdim, chunk, sink)


# ---- routed experts ---------------------------------------------------------------------------------------------------
def moe_select(z: torch.Tensor, M: int, experts: int, top: int, groups: int, keep: int, sel: torch.Tensor, wgt: torch.Tensor,
               group_top: int = 2, renorm: bool = False, softmax: bool = False, scale: float = 0.0, bias: Optional[torch.Tensor] = None):
    """sel / wgt [M][top]: the chosen experts and their weights.  Scores: sigmoid(z), or softmax(z) over all experts;
    renorm divides the chosen scores by their sum (+ 1e-20); scale (0: none) multiplies the weights."""
    a = DlMoeSelectArgs()
    a.z, a.ldz, a.M, a.experts, a.top, a.groups, a.keep = z.data_ptr(), z.stride(0), M, experts, top, groups, keep
    a.group_top, a.renorm, a.sel, a.wgt = group_top, 1 if renorm else 0, sel.data_ptr(), wgt.data_ptr()
    a.score, a.scale, a.bias = 1 if softmax else 0, scale, _p(bias)
    check_layers(layers_lib().dl_moe_select(a, _stream()), "dl_moe_select")
    lib.count_launch()


def moe_rows(w_up: torch.Tensor, w_down: torch.Tensor, x: torch.Tensor, M: int, top: int, sel: torch.Tensor, wgt: torch.Tensor,
             act: torch.Tensor, y: torch.Tensor, round_x: bool, w_gate: Optional[torch.Tensor] = None, limit: float = 0.0,
             gate_silu: bool = False):
    """w_up [experts][ff][width], w_down [experts][width][ff]; one product per (row, chosen expert) pair.  With w_gate
    (like w_up) the experts are gated: a sigma(1.702 a) (1 + b) on the products a, b clamped by `limit`, else relu(u)^2."""
    a = DlMoeArgs()
    a.w_up, a.w_down, a.wtype = w_up.data_ptr(), w_down.data_ptr(), _type(w_up)
    a.width, a.ff, a.top, a.M, a.round_x = w_up.shape[2], w_up.shape[1], top, M, 1 if round_x else 0
    a.x, a.ldx, a.sel, a.wgt = x.data_ptr(), x.stride(0), sel.data_ptr(), wgt.data_ptr()
    a.act, a.y, a.ldy = act.data_ptr(), y.data_ptr(), y.stride(0)
    a.w_gate, a.limit, a.gate_act = _p(w_gate), limit, 1 if gate_silu else 0
    check_layers(layers_lib().dl_moe_rows(a, _stream()), "dl_moe_rows")
    lib.count_launch(2)


class MoeGrouped:
    """The expert products of a routed feed-forward on the tensor cores: weight images of all experts (made once), the
    scratch of the sorted rows, and the launch sequence  plan -> gather -> grouped GEMM (relu^2) -> image -> grouped GEMM
    -> weighted combine.  Nothing returns to the host between the launches."""

    def __init__(self, w_up: torch.Tensor, w_down: torch.Tensor, top: int, max_rows: int, w_gate: Optional[torch.Tensor] = None,
                 limit: float = 0.0, gate_silu: bool = False):
        Lb = layers_lib()
        self.E, self.ff, self.width, self.top = w_up.shape[0], w_up.shape[1], w_up.shape[2], top
        dev = w_up.device
        # gated experts: gate and up rows interleaved (gate_0, up_0, gate_1, ...) in ONE image of 2 ff rows, so the first
        # grouped GEMM's epilogue sees a value's two products side by side and stores the activation
        self.gated, self.limit = w_gate is not None, limit
        self.glu_op = DENSE_GLU_SILU if gate_silu else DENSE_GLU_CLAMP
        self.n_up = self.ff
        if self.gated:
            w_up = torch.stack([w_gate, w_up], dim=2).reshape(self.E, 2 * self.ff, self.width).contiguous()
            self.n_up = 2 * self.ff
        self.up_bytes = int(Lb.dl_wh_bytes(self.n_up, _round_up(self.width, 128)))
        self.down_bytes = int(Lb.dl_wh_bytes(self.width, _round_up(self.ff, 128)))
        self.wh_up = torch.empty(self.E * self.up_bytes, dtype=torch.uint8, device=dev)
        self.wh_down = torch.empty(self.E * self.down_bytes, dtype=torch.uint8, device=dev)
        for e in range(self.E):
            check_layers(Lb.dl_wh_from_dense(w_up[e].data_ptr(), self.n_up, self.width, w_up.stride(1),
                                             self.wh_up[e * self.up_bytes:].data_ptr(), _stream()), "dl_wh_from_dense")
            check_layers(Lb.dl_wh_from_dense(w_down[e].data_ptr(), self.width, self.ff, w_down.stride(1),
                                             self.wh_down[e * self.down_bytes:].data_ptr(), _stream()), "dl_wh_from_dense")
        self.max_rows = max_rows
        self.cap = _round_up(max_rows * top + 8 * self.E, 8)
        i32 = dict(dtype=torch.int32, device=dev)
        self.cnt, self.grp = torch.zeros(self.E, **i32), torch.zeros(2 * self.E, **i32)
        self.slot_row, self.pair_pos = torch.zeros(self.cap, **i32), torch.zeros(max_rows * top, **i32)
        self.xh_in = torch.zeros(xh_bytes(self.width, self.cap), dtype=torch.uint8, device=dev)
        self.xh_act = torch.zeros(xh_bytes(self.ff, self.cap), dtype=torch.uint8, device=dev)
        self.act = torch.zeros(self.cap, self.ff, dtype=torch.float32, device=dev)
        self.yp = torch.zeros(self.cap, self.width, dtype=torch.float32, device=dev)

    def nbytes(self) -> int:
        return self.wh_up.numel() + self.wh_down.numel()

    def _gemm(self, wh, group_bytes, N, K, xh, y, M, epi, param=0.0):
        e = DlEpilogue()
        e.kind, e.n_dst, e.ld, e.dst_off = EPI_DENSE, 1, y.stride(0), 0
        e.dst[0] = y.data_ptr()
        e.dense_op, e.dense_param, e.dense_param2, e.dense_aux, e.dense_aux_ld = epi, param, 0.0, None, 0
        check_layers(layers_lib().dl_gemm_wh_tc_grouped(wh.data_ptr(), group_bytes, self.E, self.grp.data_ptr(), N, _round_up(K, 128),
                                                        xh.data_ptr(), self.cap, M, e, 2, _stream()), "dl_gemm_wh_tc_grouped")
        lib.count_launch()

    def run(self, x: torch.Tensor, M: int, sel: torch.Tensor, wgt: torch.Tensor, y: torch.Tensor):
        """x [M][width] f32, sel / wgt [M][top] -> y [M][width]."""
        Lb = layers_lib()
        assert M <= self.max_rows
        n_sorted = min(self.cap, _round_up(M * self.top + 7 * self.E, 8))          # sorted rows incl. padding, at most
        a = DlMoePlanArgs()
        a.sel, a.M, a.top, a.experts, a.cap = sel.data_ptr(), M, self.top, self.E, n_sorted
        a.cnt, a.grp, a.slot_row, a.pair_pos = self.cnt.data_ptr(), self.grp.data_ptr(), self.slot_row.data_ptr(), self.pair_pos.data_ptr()
        check_layers(Lb.dl_moe_plan(a, _stream()), "dl_moe_plan")
        check_layers(Lb.dl_xh_gather_rows(x.data_ptr(), x.stride(0), self.slot_row.data_ptr(), n_sorted, self.width, self.cap,
                                          self.xh_in.data_ptr(), _stream()), "dl_xh_gather_rows")
        if self.gated:
            self._gemm(self.wh_up, self.up_bytes, self.n_up, self.width, self.xh_in, self.act, M, self.glu_op, self.limit)
        else:
            self._gemm(self.wh_up, self.up_bytes, self.ff, self.width, self.xh_in, self.act, M, DENSE_RELU2)
        check_layers(Lb.dl_xh_from_rows(self.act.data_ptr(), self.act.stride(0), n_sorted, self.ff, self.cap, self.xh_act.data_ptr(),
                                        _stream()), "dl_xh_from_rows")
        self._gemm(self.wh_down, self.down_bytes, self.width, self.ff, self.xh_act, self.yp, M, DENSE_STORE)
        check_layers(Lb.dl_moe_combine(self.yp.data_ptr(), self.yp.stride(0), self.pair_pos.data_ptr(), wgt.data_ptr(), M, self.top,
                                       self.width, y.data_ptr(), y.stride(0), _stream()), "dl_moe_combine")
        lib.count_launch(6)


_ARGMAX_SCRATCH = {}


def argmax(logits: torch.Tensor, M: int, out: torch.Tensor):
    """out[m] = argmax(logits[m]) for the first M rows (the multi-CTA pick shared with the other engines)."""
    L = layers_lib()
    key = str(out.device)
    sc = _ARGMAX_SCRATCH.get(key)
    if sc is None:
        sc = _ARGMAX_SCRATCH[key] = torch.zeros(int(L.dl_argmax_scratch_bytes(256)), dtype=torch.uint8, device=out.device)
    vocab = logits.shape[1]
    for m0 in range(0, M, 256):
        n = min(256, M - m0)
        check_layers(L.dl_argmax(logits[m0:].data_ptr(), n, vocab, logits.stride(0), out[m0:].data_ptr(), None, 0, None, 0, 0,
                                 None, None, 0, sc.data_ptr(), 0, _stream()), "dl_argmax")
        lib.count_launch()


def sample_rows(logits: torch.Tensor, temperature, topp, coin, tokens_out):
    M, vocab = logits.shape
    check_layers(layers_lib().dl_sample_rows(logits.data_ptr(), M, vocab, logits.stride(0), temperature.data_ptr(),
                                             topp.data_ptr(), coin.data_ptr(), tokens_out.data_ptr(), _stream()),
                 "dl_sample_rows")
    lib.count_launch()
