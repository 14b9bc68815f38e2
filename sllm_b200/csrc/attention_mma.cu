// Tensor-core attention over the paged cache for the bfloat16 path: causal GQA with an
// online softmax, for prompt portions and for decoding, in one kernel family.
//
// The query heads that share a kv head are stacked along the M dimension of the MMA:
// a tile's rows are (token, head-in-group) pairs of one request and one kv head, so a
// key/value tile fetched from the pages serves all of the group's heads.  Each row
// carries its own position, so a portion that starts anywhere in the context, and a
// single decoded token, are the same code.
//
//   PREFILL form: 128 rows per CTA, 8 warps x 16 rows, every warp walks all keys of a tile.
//   DECODE form:  16 rows per CTA (a request's one or two tokens x its group); the four
//                 warps take different 16-key slices of each 64-key tile and merge at the
//                 end; the grid's z dimension splits the context further (split-KV), the
//                 partial results go to scratch and a second kernel combines them.
//
// With pooled blocks (see `AttnParams`) a CTA first walks tiles of the blocks' entries that its rows may see, then the
// window's token tiles; every row masks the entries and tokens that are not its own to see.
//
// Scores, softmax and the output accumulation are float32 (mma.sync m16n8k16, bf16 in,
// f32 out); probabilities are rounded to bfloat16 for the P.V product.
// Formulas: ref/qwen3_5.py:373-390 (scores * scale, causal mask, softmax, P.V);
// ref/standard.py:65-68 (query head h reads kv head h / group).  The reference has no
// such kernel on the device: its decode attention is one CTA per head without tensor
// cores (kernels/cuda/kernels.cu:957-1025) and its prefill runs in numpy.
#include <math.h>
#include <stdio.h>

#include "mma.cuh"

namespace sllm {

struct AttnParams {
  const __nv_bfloat16* q;        // [T, nq, HD]
  const __nv_bfloat16* k_cache;  // [pages, nkv, page_size, HD]
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;            // [T, nq, HD]
  float* part_o;                 // [splits, T, nq, HD]   (splits > 1)
  float* part_lse;               // [splits, T, nq]
  const int* block_tables;       // [S, max_pages]
  const int* q_start;            // [S+1]
  const int* ctx_len;            // [S]
  const int* tile_seq;           // [tiles]
  const int* tile_row0;          // [tiles]
  int max_pages, page_size, nq, nkv, window, num_splits, total_tokens;
  int block;     // > 0: a query sees only keys of its own block of this many positions (counted from 0)
  float scale_log2;              // scale * log2(e)
  const float* sink;             // [nq] or null: exp(sink_h) joins the softmax's denominator (no key, no value, not scaled)
  // pooled blocks beside a window (pool > 0; needs window > 0 and num_splits == 1): a query at position i also sees entry b
  // of the pooled cache (same page geometry) for every b < (i - window + 1) / pool; these entries are walked as key tiles
  // of their own before the window's
  const __nv_bfloat16* pk_cache;
  const __nv_bfloat16* pv_cache;
  const int* pool_tables;        // [S, pool_max_pages]
  int pool_max_pages, pool;
  // out_ld > 0: the output row of token t and head h is out + t * out_ld + out_off + h * vdim, vdim <= HD channels of it
  int out_ld, out_off, vdim;
  float out_scale;               // a factor on the result
};

constexpr int ATT_BN = 64;     // keys per tile
// block-table entries a CTA keeps in shared memory (the decode form reads a split of the
// context only, and must leave room for two CTAs per SM)
template <bool DECODE> struct AttBtCache { static constexpr int value = DECODE ? 512 : 1024; };
template <bool DECODE> struct AttThreads { static constexpr int value = DECODE ? 128 : 256; };
template <bool DECODE> struct AttStages { static constexpr int value = DECODE ? 3 : 4; };

template <int HD, bool DECODE>
__global__ void __launch_bounds__(AttThreads<DECODE>::value) attention_mma_kernel(const AttnParams p) {
  constexpr int NTHREADS = AttThreads<DECODE>::value;
  constexpr int STRIDE = HD + 8;                 // 16 bytes of padding: ldmatrix rows fall in distinct banks
  constexpr int KSTEPS = HD / 16;
  constexpr int DT = HD / 8;                     // output n-tiles
  constexpr int BM = DECODE ? 16 : 128;
  constexpr int NT = DECODE ? 2 : 8;             // 8-key n-tiles a warp computes per key tile
  constexpr int CHUNKS = HD / 8;                 // 16-byte chunks per row
  // key/value tiles in flight.  Both forms are bound by the latency of a tile's loads, not by their
  // bandwidth: with 2 stages the prefill form took 234 us a layer at 7B sizes, with 4 stages 160 us.
  constexpr int STAGES = AttStages<DECODE>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* k_s = q_s + BM * STRIDE;
  __nv_bfloat16* v_s = k_s + STAGES * ATT_BN * STRIDE;
  constexpr int BT_CACHE = AttBtCache<DECODE>::value;
  int* bt_s = reinterpret_cast<int*>(v_s + STAGES * ATT_BN * STRIDE);      // [BT_CACHE]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_wait();       // everything below reads what the step's earlier kernels or its batch upload wrote
  // the KV head is the grid's fastest index: tiles come longest first and CTAs start in grid order,
  // so every head's long tiles start in the first wave
  const int tile_i = blockIdx.x / p.nkv, kvh = blockIdx.x % p.nkv, split = blockIdx.z;
  const int seq = p.tile_seq[tile_i], row0 = p.tile_row0[tile_i];
  const int G = p.nq / p.nkv;
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0, ctx = p.ctx_len[seq];
  const int rows_total = q_len * G;
  const int pos0 = ctx - q_len;                  // position of the request's first token of this step
  const int row_hi = min(row0 + BM, rows_total);
  const int* bt = p.block_tables + (size_t)seq * p.max_pages;

  int key_hi = pos0 + (row_hi - 1) / G + 1;      // exclusive: the last row's own position is its last key
  int key_lo = 0;
  if (p.window > 0) key_lo = max(0, pos0 + row0 / G - p.window + 1);
  if (p.block > 0) key_lo = max(key_lo, (pos0 + row0 / G) / p.block * p.block);
  if (p.num_splits > 1 && p.out_ld == 0) {
    const int chunk = ((ctx + p.num_splits - 1) / p.num_splits + ATT_BN - 1) / ATT_BN * ATT_BN;
    key_lo = max(key_lo, split * chunk);
    key_hi = min(key_hi, (split + 1) * chunk);
  }
  const int tile0 = key_lo / ATT_BN * ATT_BN;    // tiles start at multiples of 64 keys, whatever the cut
  const int n_tok_tiles = key_hi > tile0 ? (key_hi - tile0 + ATT_BN - 1) / ATT_BN : 0;
  // pooled entries: as many as the tile's last row sees (earlier rows mask the rest)
  int nb_max = 0;
  if (p.pool > 0 && row_hi > row0) {
    const int lo_last = pos0 + (row_hi - 1) / G - p.window + 1;
    nb_max = lo_last > 0 ? lo_last / p.pool : 0;
  }
  const int n_ptiles = (nb_max + ATT_BN - 1) / ATT_BN;
  const int n_all = n_ptiles + n_tok_tiles;
  const int* pt = p.pool > 0 ? p.pool_tables + (size_t)seq * p.pool_max_pages : nullptr;
  // this CTA's share of the tiles: all of them, or (out_ld > 0: the form with its own output layout) one of num_splits
  // runs of consecutive tiles, pooled and token tiles alike
  int t_begin = 0, n_tiles = n_all;
  if (p.out_ld > 0 && p.num_splits > 1) {
    const int per = (n_all + p.num_splits - 1) / p.num_splits;
    t_begin = min(split * per, n_all);
    n_tiles = min(per, n_all - t_begin);
  }

  // the pages of this CTA's key range, fetched once: a tile's loads then depend on shared
  // memory only, not on a global load of the table
  const int page_first = tile0 / p.page_size;
  const int page_count = n_tok_tiles > 0 ? (key_hi - 1) / p.page_size - page_first + 1 : 0;
  const bool bt_cached = page_count <= BT_CACHE;
  if (bt_cached) {
    for (int i = tid; i < page_count; i += NTHREADS) bt_s[i] = bt[page_first + i];
    __syncthreads();
  }

  // ---- loads -----------------------------------------------------------------------
  auto load_q = [&]() {
    for (int c = tid; c < BM * CHUNKS; c += NTHREADS) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const int row = row0 + r;
      const bool ok = row < rows_total;
      const int tok = ok ? row / G : 0, hg = ok ? row % G : 0;
      const __nv_bfloat16* src = p.q + ((size_t)(q0 + tok) * p.nq + kvh * G + hg) * HD + ch * 8;
      cp_async_16(q_s + r * STRIDE + ch * 8, src, ok);
    }
  };
  // each thread keeps one 16-byte column of the rows r_first, r_first + R_STEP, ...: the address
  // arithmetic of a tile is a handful of instructions per row
  constexpr int R_STEP = NTHREADS / CHUNKS;
  const int ch8 = (tid % CHUNKS) * 8, r_first = tid / CHUNKS;
  const int ps = p.page_size;
  const int ps_shift = (ps & (ps - 1)) == 0 ? __ffs(ps) - 1 : -1;
  const size_t head_off = (size_t)kvh * ps * HD + ch8;
  const size_t page_stride = (size_t)p.nkv * ps * HD;
  auto load_kv = [&](int tile, int buf) {
    tile += t_begin;
    if (tile < n_ptiles) {                        // a tile of pooled entries
#pragma unroll
      for (int r = r_first; r < ATT_BN; r += R_STEP) {
        const int e = tile * ATT_BN + r;
        bool ok = e < nb_max;
        int page = 0, off = 0;
        if (ok) {
          const int pi = ps_shift >= 0 ? e >> ps_shift : e / ps;
          off = e - pi * ps;
          page = pi < p.pool_max_pages ? pt[pi] : -1;
          ok = page >= 0;
          if (!ok) page = 0;
        }
        const size_t src = (size_t)page * page_stride + head_off + (size_t)off * HD;
        cp_async_16(k_s + (buf * ATT_BN + r) * STRIDE + ch8, p.pk_cache + src, ok);
        cp_async_16(v_s + (buf * ATT_BN + r) * STRIDE + ch8, p.pv_cache + src, ok);
      }
      return;
    }
    const int kbase = tile0 + (tile - n_ptiles) * ATT_BN;
#pragma unroll
    for (int r = r_first; r < ATT_BN; r += R_STEP) {
      const int key = kbase + r;
      bool ok = key < key_hi && key >= key_lo;
      int page = 0, off = 0;
      if (ok) {
        const int pi = ps_shift >= 0 ? key >> ps_shift : key / ps;
        off = key - pi * ps;
        page = bt_cached ? bt_s[pi - page_first] : bt[pi];
        ok = page >= 0;                           // a page given back is never read
        if (!ok) page = 0;
      }
      const size_t src = (size_t)page * page_stride + head_off + (size_t)off * HD;
      cp_async_16(k_s + (buf * ATT_BN + r) * STRIDE + ch8, p.k_cache + src, ok);
      cp_async_16(v_s + (buf * ATT_BN + r) * STRIDE + ch8, p.v_cache + src, ok);
    }
  };

  load_q();
  cp_async_commit();
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles) load_kv(st, st);
    cp_async_commit();
  }

  // ---- per-thread rows: g and g+8 of the warp's 16-row block ---------------------------
  const int wrow = DECODE ? 0 : warp * 16;
  int hi_r[2], lo_r[2], nb_r[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + g + 8 * i;
    nb_r[i] = 0;
    if (row < rows_total) {
      const int pos = pos0 + row / G;
      if (p.pool > 0 && pos - p.window + 1 > 0) nb_r[i] = (pos - p.window + 1) / p.pool;
      hi_r[i] = min(pos + 1, key_hi);
      lo_r[i] = p.window > 0 ? max(key_lo, pos - p.window + 1) : key_lo;
      if (p.block > 0) lo_r[i] = max(lo_r[i], pos / p.block * p.block);
    } else {
      hi_r[i] = 0;
      lo_r[i] = 1;                                // empty
    }
  }
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[d][c] = 0.f;

  cp_async_wait<STAGES - 1>();                    // the queries have landed
  __syncthreads();
  unsigned qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldmatrix_x4(qf[ks], q_s + (wrow + (lane & 15)) * STRIDE + ks * 16 + (lane >> 4) * 8);

  const int koff = DECODE ? warp * 16 : 0;        // the warp's keys within a tile
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile % STAGES;
    if (tile + STAGES - 1 < n_tiles) load_kv(tile + STAGES - 1, (tile + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();                  // tile `tile` has landed
    __syncthreads();
    const __nv_bfloat16* kb = k_s + buf * ATT_BN * STRIDE;
    const __nv_bfloat16* vb = v_s + buf * ATT_BN * STRIDE;

    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        unsigned b[4];
        ldmatrix_x4(b, kb + (koff + n * 8 + (lane >> 4) * 8 + (lane & 7)) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[n], qf[ks], b[0], b[1]);
        mma_bf16(s[n + 1], qf[ks], b[2], b[3]);
      }
    }
    // mask, scale (into the log2 domain), row maxima
    const int vtile = t_begin + tile;
    const bool pooled_tile = vtile < n_ptiles;
    const int kbase = (pooled_tile ? vtile * ATT_BN : tile0 + (vtile - n_ptiles) * ATT_BN) + koff;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = kbase + n * 8 + 2 * t4 + (c & 1);
        const int i = c >> 1;
        const bool seen = pooled_tile ? key < nb_r[i] : (key < hi_r[i] && key >= lo_r[i]);
        const float v = seen ? s[n][c] * p.scale_log2 : -INFINITY;
        s[n][c] = v;
        mx[i] = fmaxf(mx[i], v);
      }
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m_r[i], mx[i]);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;    // a row with no key yet
      corr[i] = exp2f(m_r[i] - m_use);
      m_r[i] = m_new;
      mx[i] = m_use;
      l_r[i] *= corr[i];
    }
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= corr[0]; o[d][1] *= corr[0];
      o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
    unsigned pf[NT / 2][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const float p0 = exp2f(s[n][0] - mx[0]), p1 = exp2f(s[n][1] - mx[0]);
      const float p2 = exp2f(s[n][2] - mx[1]), p3 = exp2f(s[n][3] - mx[1]);
      l_r[0] += p0 + p1;
      l_r[1] += p2 + p3;
      pf[n / 2][(n & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[n / 2][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vb + (koff + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + d * 8 + (lane >> 4) * 8);
        mma_bf16(o[d], pf[kk], b[0], b[1]);
        mma_bf16(o[d + 1], pf[kk], b[2], b[3]);
      }
    }
    __syncthreads();                              // the next iteration refills the buffer just read
  }
  cp_async_wait<0>();
  pdl_launch_dependents();             // all keys are read; the next kernel may begin during the epilogue

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 1);
    l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 2);
  }

  if constexpr (!DECODE) {
    // each warp owns its rows
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + wrow + g + 8 * i;
      if (row >= rows_total) continue;
      const size_t orow = (size_t)(q0 + row / G) * p.nq + kvh * G + row % G;
      if (p.sink != nullptr && p.num_splits == 1) l_r[i] += exp2f(p.sink[kvh * G + row % G] * 1.4426950408889634f - m_r[i]);
      const float inv = l_r[i] > 0.f ? (p.num_splits > 1 ? 1.f : p.out_scale) / l_r[i] : 0.f;
      if (p.out_ld > 0 && p.num_splits == 1) {
        __nv_bfloat16* po = p.out + (size_t)(q0 + row / G) * p.out_ld + p.out_off + (size_t)(kvh * G + row % G) * p.vdim;
#pragma unroll
        for (int d = 0; d < DT; ++d)
          if (d * 8 + 2 * t4 < p.vdim)
            *reinterpret_cast<unsigned*>(po + d * 8 + 2 * t4) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
      } else if (p.num_splits > 1) {
        float* po = p.part_o + ((size_t)split * p.total_tokens * p.nq + orow) * HD;
#pragma unroll
        for (int d = 0; d < DT; ++d)
          *reinterpret_cast<float2*>(po + d * 8 + 2 * t4) = make_float2(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
        if (t4 == 0)
          p.part_lse[(size_t)split * p.total_tokens * p.nq + orow] = l_r[i] > 0.f ? m_r[i] + log2f(l_r[i]) : -INFINITY;
      } else {
        __nv_bfloat16* po = p.out + orow * HD;
#pragma unroll
        for (int d = 0; d < DT; ++d)
          *reinterpret_cast<unsigned*>(po + d * 8 + 2 * t4) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
      }
    }
  } else {
    // the four warps hold partial results for the same 16 rows over different keys: merge
    float* mo = reinterpret_cast<float*>(k_s);                 // [4][16][HD]
    float* mm = mo + 4 * 16 * HD;                              // [4][16] maxima, then [4][16] sums
    float* ml = mm + 64;
    static_assert(sizeof(float) * (4 * 16 * HD + 128) <= sizeof(__nv_bfloat16) * 2 * STAGES * ATT_BN * STRIDE, "merge buffer");
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = g + 8 * i;
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<float2*>(mo + (warp * 16 + r) * HD + d * 8 + 2 * t4) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
      if (t4 == 0) {
        mm[warp * 16 + r] = m_r[i];
        ml[warp * 16 + r] = l_r[i];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < 16 * (HD / 4); idx += 128) {
      const int r = idx / (HD / 4), d4 = (idx % (HD / 4)) * 4;
      const int row = row0 + r;
      if (row >= rows_total) continue;
      float mt = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mt = fmaxf(mt, mm[w * 16 + r]);
      float lt = 0.f, f[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        f[w] = ml[w * 16 + r] > 0.f ? exp2f(mm[w * 16 + r] - mt) : 0.f;
        lt += ml[w * 16 + r] * f[w];
      }
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * HD + d4);
        acc.x += v.x * f[w]; acc.y += v.y * f[w]; acc.z += v.z * f[w]; acc.w += v.w * f[w];
      }
      if (p.sink != nullptr && p.num_splits == 1) lt += exp2f(p.sink[kvh * G + row % G] * 1.4426950408889634f - mt);
      const float inv = lt > 0.f ? (p.num_splits > 1 ? 1.f : p.out_scale) / lt : 0.f;
      const size_t orow = (size_t)(q0 + row / G) * p.nq + kvh * G + row % G;
      if (p.out_ld > 0 && p.num_splits == 1) {
        if (d4 < p.vdim) {
          __nv_bfloat16* po = p.out + (size_t)(q0 + row / G) * p.out_ld + p.out_off + (size_t)(kvh * G + row % G) * p.vdim + d4;
          *reinterpret_cast<uint2*>(po) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
      } else if (p.num_splits > 1) {
        float* po = p.part_o + ((size_t)split * p.total_tokens * p.nq + orow) * HD + d4;
        *reinterpret_cast<float4*>(po) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        if (d4 == 0) p.part_lse[(size_t)split * p.total_tokens * p.nq + orow] = lt > 0.f ? mt + log2f(lt) : -INFINITY;
      } else {
        __nv_bfloat16* po = p.out + orow * HD + d4;
        *reinterpret_cast<uint2*>(po) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
      }
    }
  }
}

// out[row] = sum_s w_s part_o[s][row], w_s = 2^(lse_s - max) / sum: the splits of one row merged.
template <int HD>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                             __nv_bfloat16* __restrict__ out, int rows, int num_splits,
                                             const int* __restrict__ tile_seq, const int* __restrict__ q_start, int nq,
                                             const float* __restrict__ sink, int out_ld, int out_off, int vdim, float out_scale) {
  // One CTA per (tile, query head, token of the tile's request): the rows the decode form wrote and no others, so
  // that a step's other rows (a prompt portion's, the prefill form's) are neither read nor touched.  The step's
  // description is read before the wait for the kernel before.
  const int seq = tile_seq[blockIdx.x];
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  pdl_launch_dependents();       // a short kernel: the successor may be set up behind it
  pdl_wait();
  if ((int)blockIdx.z >= q_len) return;
  const int row = (q0 + (int)blockIdx.z) * nq + (int)blockIdx.y;
  float mt = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mt = fmaxf(mt, part_lse[(size_t)s * rows + row]);
  float tot = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float l = part_lse[(size_t)s * rows + row];
    tot += l == -INFINITY ? 0.f : exp2f(l - mt);
  }
  if (sink != nullptr) tot += exp2f(sink[blockIdx.y] * 1.4426950408889634f - mt);
  const float inv = tot > 0.f ? out_scale / tot : 0.f;
  // (out_ld > 0: the row of token t and head h lies at out + t * out_ld + out_off + h * vdim and holds vdim channels)
  __nv_bfloat16* po = out_ld > 0 ? out + (size_t)(q0 + (int)blockIdx.z) * out_ld + out_off + (size_t)blockIdx.y * vdim : out + (size_t)row * HD;
  const int lim = out_ld > 0 ? vdim : HD;
  for (int d = threadIdx.x; d < lim; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float l = part_lse[(size_t)s * rows + row];
      if (l != -INFINITY) acc += part_o[((size_t)s * rows + row) * HD + d] * exp2f(l - mt);
    }
    po[d] = __float2bfloat16_rn(acc * inv);
  }
}

template <int HD, bool DECODE>
static int launch_attention(const AttnParams& p, int tiles, cudaStream_t stream) {
  constexpr int BM = DECODE ? 16 : 128;
  constexpr size_t smem = sizeof(__nv_bfloat16) * (size_t)(BM + 2 * AttStages<DECODE>::value * ATT_BN) * (HD + 8) +
                          sizeof(int) * AttBtCache<DECODE>::value;
  static bool configured = false;                 // per template instance
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, DECODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_error("attention_mma: cannot raise the shared memory limit");
      return SLLM_ERR_LAUNCH;
    }
    configured = true;
  }
  dim3 grid((unsigned)tiles * p.nkv, 1, p.num_splits);
  launch_kernel(attention_mma_kernel<HD, DECODE>, grid, AttThreads<DECODE>::value, smem, stream, p);
  int rc = launch_status("attention_mma");
  if (rc != SLLM_OK) return rc;
  if (p.num_splits > 1) {
    const int G = p.nq / p.nkv;
    launch_kernel(attention_combine_kernel<HD>, dim3((unsigned)tiles, (unsigned)p.nq, (unsigned)(16 / G > 0 ? 16 / G : 1)), HD >= 128 ? 128 : 64, 0, stream,
                  (const float*)p.part_o, (const float*)p.part_lse, p.out, p.total_tokens * p.nq, p.num_splits, p.tile_seq,
                  p.q_start, p.nq, p.sink, p.out_ld, p.out_off, p.vdim, p.out_scale);
    rc = launch_status("attention_combine");
  }
  return rc;
}

}  // namespace sllm

using namespace sllm;

// 1 if the tensor-core kernel takes this head size (others go to the CUDA-core kernel).
SLLM_EXPORT int sllm_attention_mma_supports(int hd) { return hd == 16 || hd == 32 || hd == 64 || hd == 128; }

// tiles: tile_seq/tile_row0 [tiles] describe 128-row (decode == 0) or 16-row (decode == 1) tiles of
// (token, head-in-group) rows.  part_o/part_lse are scratch for num_splits > 1:
// float32 [num_splits, T, nq, hd] and [num_splits, T, nq].
SLLM_EXPORT int sllm_attention_mma(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                                   float* part_lse, const int* block_tables, int max_pages, const int* q_start,
                                   const int* ctx_len, const int* tile_seq, const int* tile_row0, int tiles,
                                   int decode, int num_splits, int total_tokens, int nq, int nkv, int hd,
                                   int page_size, float scale, int window, int block, const float* sink, cudaStream_t stream) {
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_mma: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_mma_supports(hd), "attention_mma: head_dim=%d is not one of 16, 32, 64, 128", hd);
  SLLM_REQUIRE(page_size > 0 && max_pages > 0 && tiles >= 0 && total_tokens >= 0, "attention_mma: bad sizes");
  SLLM_REQUIRE(num_splits >= 1 && num_splits <= 65535 && nkv <= 65535, "attention_mma: bad grid nkv=%d splits=%d", nkv, num_splits);
  SLLM_REQUIRE(num_splits == 1 || (part_o && part_lse), "attention_mma: split-KV needs scratch");
  if (tiles == 0) return SLLM_OK;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_lse = part_lse; p.block_tables = block_tables;
  p.q_start = q_start; p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
  p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.window = window; p.block = block;
  p.num_splits = num_splits; p.total_tokens = total_tokens;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sink = sink;
  p.pk_cache = p.pv_cache = nullptr; p.pool_tables = nullptr; p.pool_max_pages = p.pool = 0;
  p.out_ld = p.out_off = p.vdim = 0; p.out_scale = 1.f;
#define DISPATCH(HD_)                                                             \
  case HD_:                                                                       \
    return decode ? launch_attention<HD_, true>(p, tiles, stream) : launch_attention<HD_, false>(p, tiles, stream);
  switch (hd) {
    DISPATCH(16) DISPATCH(32) DISPATCH(64) DISPATCH(128)
  }
#undef DISPATCH
  return SLLM_ERR_UNSUPPORTED;
}

// The same kernels over a window of tokens plus pooled blocks (see `AttnParams`); the result, times `out_scale`, goes to
// columns out_off + h * vdim of rows of `out_ld` elements.  The 16-row form may cut its tiles (pooled and token tiles
// alike) into `num_splits` runs that CTAs of their own walk; the merge kernel then writes the rows.
SLLM_EXPORT int sllm_attention_mma_pooled(const void* q, const void* k_cache, const void* v_cache, const void* pk_cache,
                                          const void* pv_cache, void* out, const int* block_tables, int max_pages,
                                          const int* pool_tables, int pool_max_pages, const int* q_start, const int* ctx_len,
                                          const int* tile_seq, const int* tile_row0, int tiles, int decode, int num_splits,
                                          float* part_o, float* part_lse, int total_tokens,
                                          int nq, int nkv, int hd, int vdim, int page_size, float scale, int window, int pool,
                                          const float* sink, float out_scale, int out_ld, int out_off, cudaStream_t stream) {
  SLLM_REQUIRE(num_splits >= 1 && num_splits <= 65535 && (num_splits == 1 || (decode && part_o && part_lse)),
               "attention_mma_pooled: %d runs of tiles need the 16-row form and scratch", num_splits);
  SLLM_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_mma_pooled: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(sllm_attention_mma_supports(hd), "attention_mma_pooled: head_dim=%d is not one of 16, 32, 64, 128", hd);
  SLLM_REQUIRE(page_size > 0 && max_pages > 0 && tiles >= 0 && total_tokens >= 0 && nkv <= 65535, "attention_mma_pooled: bad sizes");
  if (pool_max_pages <= 0) pool = 0;              // no request of the step holds an entry yet
  SLLM_REQUIRE(pool == 0 || (window > 0 && pool_tables && pk_cache && pv_cache),
               "attention_mma_pooled: pooled entries need a window, their pages and their tables");
  SLLM_REQUIRE(vdim > 0 && vdim <= hd && vdim % 4 == 0 && out_ld % 4 == 0 && out_off % 4 == 0 && out_off >= 0 &&
                   out_off + nq * vdim <= out_ld && ((uintptr_t)out & 7) == 0,
               "attention_mma_pooled: the output's columns (%d heads of %d from %d in rows of %d) must be multiples of 4", nq, vdim, out_off, out_ld);
  if (tiles == 0) return SLLM_OK;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_lse = part_lse; p.block_tables = block_tables;
  p.q_start = q_start; p.ctx_len = ctx_len; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
  p.max_pages = max_pages; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.window = window; p.block = 0;
  p.num_splits = num_splits; p.total_tokens = total_tokens;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sink = sink;
  p.pk_cache = (const __nv_bfloat16*)pk_cache; p.pv_cache = (const __nv_bfloat16*)pv_cache; p.pool_tables = pool_tables;
  p.pool_max_pages = pool_max_pages; p.pool = pool;
  p.out_ld = out_ld; p.out_off = out_off; p.vdim = vdim; p.out_scale = out_scale;
#define DISPATCH(HD_)                                                             \
  case HD_:                                                                       \
    return decode ? launch_attention<HD_, true>(p, tiles, stream) : launch_attention<HD_, false>(p, tiles, stream);
  switch (hd) {
    DISPATCH(16) DISPATCH(32) DISPATCH(64) DISPATCH(128)
  }
#undef DISPATCH
  return SLLM_ERR_UNSUPPORTED;
}
