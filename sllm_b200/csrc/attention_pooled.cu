// Attention over a window of recent tokens plus one pooled key and value per block of older tokens.
//
//   Query at position i sees the keys j with 0 <= i - j < window (from the token cache) and, beside them, entry b of
//   the pooled cache for every block b of `pool` positions that lies wholly before the window:
//   b * pool + pool - 1 <= i - window, that is b < (i - window + 1) / pool.  Entry b is the mean of the block's keys as
//   the token cache holds them, and of its values.  Tokens and blocks share one softmax; with `sink` (a number per query
//   head) its denominator also holds exp(sink_h).  window <= 0: every earlier token is seen and no block.
//
//   pool_kv_write            the token that completes a block (its place in the pooled pages comes with the step's
//                            description, -1 for every other token) reads the block's keys and values from the token
//                            pages, adds them in float32 (in an order that depends on the block's length alone) and
//                            writes their means.
//   attention_pooled_simt    CUDA cores, float32 arithmetic, one CTA per (token, query head): any head size up to 256,
//                            float32 or bfloat16 caches.  Prompt portions and single decoded tokens are the same work.
//   (bfloat16 heads of 16, 32, 64 or 128 channels run on the tensor cores instead: the mma.sync forms of
//   attention_mma.cu walk tiles of the blocks' entries in front of the window's token tiles.)
//
// Each warp of the CUDA-core form takes the row's keys w, w+W, w+2W, ... (pooled entries first, then tokens) in ascending
// order with an online softmax; the warps' partial results are merged in warp order.  The order depends on the position
// alone.
#include <math.h>

#include "common.cuh"

namespace sllm {

constexpr int AP_WARPS = 4;
constexpr int AP_MAX_D = 256;

constexpr int PW_WARPS = 8;

__device__ __forceinline__ void pw_add(float* acc, const uint4& raw, float) {
  acc[0] += __uint_as_float(raw.x); acc[1] += __uint_as_float(raw.y); acc[2] += __uint_as_float(raw.z); acc[3] += __uint_as_float(raw.w);
}
__device__ __forceinline__ void pw_add(float* acc, const uint4& raw, __nv_bfloat16) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    acc[2 * k] += f.x;
    acc[2 * k + 1] += f.y;
  }
}

// grid (T, nkv), 8 warps: warp w adds the block's tokens w, w+8, w+16, ... in ascending order, then the warps' sums are
// added in warp order: the order depends on the block's length alone.  A lane holds 16 bytes of a row (VEC: rows whose
// length is a multiple of that; else one channel), so a warp's load instruction fetches a whole row of up to 256 bfloat16
// channels, and the loads of eight rows are in flight together: a block of 64 tokens is two round trips to memory.
template <typename TC, bool VEC>
__global__ void __launch_bounds__(PW_WARPS * 32)
pool_kv_write_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache, const int* __restrict__ block_tables,
                     int max_pages, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                     const int* __restrict__ pool_slots, TC* __restrict__ pk_cache, TC* __restrict__ pv_cache, int pool_pages,
                     int nkv, int D, int page_size, int pool) {
  extern __shared__ float pw_sm[];               // [2][PW_WARPS][D]
  constexpr int E = VEC ? 16 / (int)sizeof(TC) : 1;
  constexpr int U = 8;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, kvh = blockIdx.y;
  const int slot = pool_slots[t];
  if (slot < 0 || slot / page_size >= pool_pages) return;
  const int pos = positions[t];
  const int* bt = block_tables + (size_t)seq_of_token[t] * max_pages;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int first = pos - pool + 1;
  for (int d0 = 0; d0 < D; d0 += 32 * E) {
    const int d = d0 + lane * E;
    float sk[E], sv[E];
#pragma unroll
    for (int e = 0; e < E; ++e) sk[e] = sv[e] = 0.f;
    for (int i0 = warp; i0 < pool; i0 += PW_WARPS * U) {
      size_t row[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u * PW_WARPS, j = first + i;
        const int page = (i < pool && j >= 0) ? bt[j / page_size] : -1;
        ok[u] = page >= 0 && d < D;
        row[u] = ok[u] ? (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * D + d : 0;
      }
      if constexpr (VEC) {
        uint4 kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          kk[u] = ok[u] ? *reinterpret_cast<const uint4*>(k_cache + row[u]) : make_uint4(0u, 0u, 0u, 0u);
          vv[u] = ok[u] ? *reinterpret_cast<const uint4*>(v_cache + row[u]) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          pw_add(sk, kk[u], TC());
          pw_add(sv, vv[u], TC());
        }
      } else {
        float kk[U], vv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          kk[u] = ok[u] ? to_f32(k_cache[row[u]]) : 0.f;
          vv[u] = ok[u] ? to_f32(v_cache[row[u]]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          sk[0] += kk[u];
          sv[0] += vv[u];
        }
      }
    }
    if (d < D) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        pw_sm[warp * D + d + e] = sk[e];
        pw_sm[(PW_WARPS + warp) * D + d + e] = sv[e];
      }
    }
  }
  __syncthreads();
  const size_t dst = (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sk = 0.f, sv = 0.f;
#pragma unroll
    for (int w = 0; w < PW_WARPS; ++w) {
      sk += pw_sm[w * D + d];
      sv += pw_sm[(PW_WARPS + w) * D + d];
    }
    pk_cache[dst + d] = from_f32<TC>(sk / (float)pool);
    pv_cache[dst + d] = from_f32<TC>(sv / (float)pool);
  }
}

template <typename TC>
__global__ void __launch_bounds__(AP_WARPS * 32)
attention_pooled_simt_kernel(const TC* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                             const TC* __restrict__ pk_cache, const TC* __restrict__ pv_cache,
                             const int* __restrict__ block_tables, int max_pages, const int* __restrict__ pool_tables,
                             int pool_max_pages, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                             int nq, int nkv, int D, int vdim, int page_size, float scale, int window, int pool,
                             const float* __restrict__ sink, float out_scale, TC* __restrict__ out, int out_ld, int out_off) {
  __shared__ float qs[AP_MAX_D];
  __shared__ float acc_s[AP_WARPS][AP_MAX_D];
  __shared__ float m_s[AP_WARPS], l_s[AP_WARPS];
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int kvh = h / (nq / nkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = positions[t];
  const int seq = seq_of_token[t];
  const int* bt = block_tables + (size_t)seq * max_pages;
  const int* pt = pool_tables != nullptr ? pool_tables + (size_t)seq * pool_max_pages : nullptr;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int nb = (window > 0 && pool > 0 && pt != nullptr) ? lo / pool : 0;        // blocks wholly before the window
  const int total = nb + (pos - lo + 1);

  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = to_f32(q[((size_t)t * nq + h) * D + d]);
  __syncthreads();

  float acc[AP_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < AP_MAX_D / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int n = warp; n < total; n += AP_WARPS) {
    const TC* kr;
    const TC* vr;
    if (n < nb) {
      const int page = n / page_size < pool_max_pages ? pt[n / page_size] : -1;
      if (page < 0) continue;
      const size_t row = (((size_t)page * nkv + kvh) * page_size + (n % page_size)) * D;
      kr = pk_cache + row;
      vr = pv_cache + row;
    } else {
      const int j = lo + (n - nb);
      const int page = bt[j / page_size];
      if (page < 0) continue;                          // never dereference a page that was given back
      const size_t row = (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * D;
      kr = k_cache + row;
      vr = v_cache + row;
    }
    float dot = 0.f;
    for (int d = lane; d < D; d += 32) dot = fmaf(qs[d], to_f32(kr[d]), dot);
    dot = warp_sum(dot);
    const float s = dot * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);              // exp(-inf) = 0 on the first key
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < AP_MAX_D / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < vdim) acc[i] = acc[i] * corr + p * to_f32(vr[d]);
    }
    m = m_new;
  }
  if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
  for (int i = 0; i < AP_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) acc_s[warp][d] = acc[i];
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < AP_WARPS; ++w) mm = fmaxf(mm, m_s[w]);
  if (sink != nullptr) mm = fmaxf(mm, sink[h]);        // the sink may be the largest term: keep every exponent <= 0
  float ll = 0.f;
  float f[AP_WARPS];
#pragma unroll
  for (int w = 0; w < AP_WARPS; ++w) {
    f[w] = l_s[w] > 0.f ? expf(m_s[w] - mm) : 0.f;
    ll += l_s[w] * f[w];
  }
  if (sink != nullptr) ll += expf(sink[h] - mm);       // a term of the denominator without key or value, not scaled
  const float inv = ll > 0.f ? out_scale / ll : 0.f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < AP_WARPS; ++w) o += acc_s[w][d] * f[w];
    out[(size_t)t * out_ld + out_off + (size_t)h * vdim + d] = from_f32<TC>(o * inv);
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_pool_kv_write(const void* k_cache, const void* v_cache, int dtype, const int* block_tables, int max_pages,
                                   const int* positions, const int* seq_of_token, const int* pool_slots, void* pk_cache,
                                   void* pv_cache, int pool_pages, int T, int nkv, int D, int page_size, int pool,
                                   cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && nkv > 0 && D > 0 && page_size > 0 && max_pages > 0 && pool > 0 && pool_pages >= 0,
               "pool_kv_write: bad sizes T=%d nkv=%d D=%d page_size=%d pool=%d", T, nkv, D, page_size, pool);
  SLLM_REQUIRE(nkv <= 65535, "pool_kv_write: %d kv heads exceed one launch", nkv);
  if (T == 0 || pool_pages == 0) return SLLM_OK;
  const dim3 grid(T, nkv);
  const size_t smem = 2 * (size_t)PW_WARPS * D * sizeof(float);
  SLLM_REQUIRE(smem <= 48 * 1024, "pool_kv_write: a head of %d channels is more than the kernel keeps in shared memory", D);
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = aligned(k_cache) && aligned(v_cache) && D % (dtype == SLLM_F32 ? 4 : 8) == 0;
#define SLLM_PW(TC, VEC_)                                                                                                      \
  launch_kernel(pool_kv_write_kernel<TC, VEC_>, grid, PW_WARPS * 32, smem, stream, (const TC*)k_cache, (const TC*)v_cache,      \
                block_tables, max_pages, positions, seq_of_token, pool_slots, (TC*)pk_cache, (TC*)pv_cache, pool_pages, nkv, D, \
                page_size, pool)
  if (dtype == SLLM_F32) { if (vec) SLLM_PW(float, true); else SLLM_PW(float, false); }
  else if (dtype == SLLM_BF16) { if (vec) SLLM_PW(__nv_bfloat16, true); else SLLM_PW(__nv_bfloat16, false); }
  else SLLM_REQUIRE(false, "pool_kv_write: unknown dtype %d", dtype);
#undef SLLM_PW
  return launch_status("pool_kv_write");
}

SLLM_EXPORT int sllm_attention_pooled_simt(const void* q, const void* k_cache, const void* v_cache, const void* pk_cache,
                                           const void* pv_cache, int dtype, const int* block_tables, int max_pages,
                                           const int* pool_tables, int pool_max_pages, const int* positions,
                                           const int* seq_of_token, int T, int nq, int nkv, int D, int vdim, int page_size,
                                           float scale, int window, int pool, const float* sink, float out_scale, void* out,
                                           int out_ld, int out_off, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention_pooled: bad head counts nq=%d nkv=%d", nq, nkv);
  SLLM_REQUIRE(D > 0 && D <= AP_MAX_D && vdim > 0 && vdim <= D, "attention_pooled: a head of %d channels (values of %d) is outside 1..%d", D, vdim, AP_MAX_D);
  SLLM_REQUIRE(page_size > 0 && max_pages > 0, "attention_pooled: bad page_size=%d max_pages=%d", page_size, max_pages);
  SLLM_REQUIRE(pool_tables == nullptr || (pool > 0 && window > 0 && pool_max_pages >= 0 && pk_cache && pv_cache),
               "attention_pooled: pooled entries need a block size, a window and their pages");
  SLLM_REQUIRE(out_off >= 0 && out_off + nq * vdim <= out_ld, "attention_pooled: the output's columns lie outside its %d", out_ld);
  SLLM_REQUIRE(nq <= 65535, "attention_pooled: %d query heads exceed one launch", nq);
  if (T == 0) return SLLM_OK;
  if (pool_max_pages == 0) pool_tables = nullptr;
  const dim3 grid(T, nq);
#define SLLM_AP(TC)                                                                                                              \
  launch_kernel(attention_pooled_simt_kernel<TC>, grid, AP_WARPS * 32, 0, stream, (const TC*)q, (const TC*)k_cache,              \
                (const TC*)v_cache, (const TC*)pk_cache, (const TC*)pv_cache, block_tables, max_pages, pool_tables, pool_max_pages, \
                positions, seq_of_token, nq, nkv, D, vdim, page_size, scale, window, pool, sink, out_scale, (TC*)out, out_ld, out_off)
  if (dtype == SLLM_F32) SLLM_AP(float);
  else if (dtype == SLLM_BF16) SLLM_AP(__nv_bfloat16);
  else SLLM_REQUIRE(false, "attention_pooled: unknown dtype %d", dtype);
#undef SLLM_AP
  return launch_status("attention_pooled_simt");
}
