// Kernels of layers that wrap each sublayer in two norms, and of the small recurrent and gated units such layers hold.
//
//   * post_add_norm: a sublayer's output is normed BEFORE it joins the stream, and the stream is normed for the next
//     reader in the same pass:  stream += term / rms(term) * post_gain;  h = stream / rms(stream) * pre_gain.  Either
//     half may be absent (the first norm of a model has no term; the last sublayer has no reader).  A CTA per token,
//     float32 throughout; `term` may be a stack of k-split partial sums.
//   * mingru_scan: the element-wise recurrence S <- (1 - z) S + z c with z = sigmoid(a), c = b + 1/2 where b >= 0 and
//     sigmoid(b) elsewhere, read out as S * silu(g); a, b, g are float32 columns of one product.  The recurrence is
//     linear in S, so a request's portion is cut into as many runs of tokens as the CTA has warps: every warp first
//     folds its run into (product of the keeps, state reached from zero), the runs' entry states follow from the
//     request's slot in a short serial pass, then every warp walks its run again from its entry state and writes.
//   * gated_clamp_act: y = g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit), gate and
//     up columns alternating in blocks; optionally times a routing weight per (token, expert) that a mixture of
//     experts carries on its activation rows (zero: not chosen, and the columns are not read).
//   * moe_route_top_softmax: the `top` largest router logits win; their weights are the softmax over the winners alone.
//   * rope_cols: per head, a few columns of a float32 product rotated by position (rotate-half layout) and written
//     into a slice of wider per-head rows (the rotated part of a query that otherwise lives in a latent space).
#include <math.h>

#include "common.cuh"

namespace sllm {

__device__ __forceinline__ float sw_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename TO>
__global__ void __launch_bounds__(256)
post_add_norm_kernel(float* __restrict__ stream, const float* __restrict__ term, int parts, size_t part_stride,
                     const float* __restrict__ post_gain, float post_eps, const float* __restrict__ pre_gain, float pre_eps,
                     TO* __restrict__ h, int W) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float* x = stream + base;
  float ss = 0.f;
  if (term != nullptr) {
    float st = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = term[base + i];
      for (int p = 1; p < parts; ++p) v += term[p * part_stride + base + i];
      st = fmaf(v, v, st);
    }
    st = block_sum(st, red);
    const float inv = 1.0f / sqrtf(st / (float)W + post_eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = term[base + i];
      for (int p = 1; p < parts; ++p) v += term[p * part_stride + base + i];
      const float y = x[i] + v * inv * post_gain[i];
      x[i] = y;
      ss = fmaf(y, y, ss);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  }
  if (h == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) h[base + i] = from_f32<TO>(x[i] * inv * pre_gain[i]);
}

constexpr int MG_WARPS = 16;

// grid (S, ceil(C / 32)), 32 * MG_WARPS threads: lane = channel, warp = run of tokens
template <typename TO>
__global__ void __launch_bounds__(32 * MG_WARPS)
mingru_scan_kernel(const float* __restrict__ proj, int ld, int off_z, int off_x, int off_g, float* __restrict__ state,
                   const int* __restrict__ q_start, const int* __restrict__ state_slots, TO* __restrict__ out, int C) {
  __shared__ float keep_s[MG_WARPS][32], reach_s[MG_WARPS][32];
  pdl_wait();
  const int seq = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.y * 32 + lane;
  const bool live = c < C;
  const int first = q_start[seq], n = q_start[seq + 1] - first;
  const int per = (n + MG_WARPS - 1) / MG_WARPS;
  const int lo = min(n, warp * per), hi = min(n, lo + per);
  float* slot = state + (size_t)state_slots[seq] * C + c;
  float S = live ? *slot : 0.f;                  // read before the barrier: the last run's warp writes it at its end
  float keep = 1.f, reach = 0.f;
  if (live && n > 1) {
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
      const float* row = proj + (size_t)(first + t) * ld + c;
      const float z = sw_sigmoid(row[off_z]), b = row[off_x];
      const float cand = b >= 0.f ? b + 0.5f : sw_sigmoid(b);
      keep *= 1.0f - z;
      reach = fmaf(1.0f - z, reach, z * cand);
    }
  }
  keep_s[warp][lane] = keep;
  reach_s[warp][lane] = reach;
  __syncthreads();
  for (int w = 0; w < warp; ++w) S = fmaf(keep_s[w][lane], S, reach_s[w][lane]);       // this run's entry state
  if (live) {
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
      const float* row = proj + (size_t)(first + t) * ld + c;
      const float z = sw_sigmoid(row[off_z]), b = row[off_x], g = row[off_g];
      const float cand = b >= 0.f ? b + 0.5f : sw_sigmoid(b);
      S = fmaf(1.0f - z, S, z * cand);
      out[(size_t)(first + t) * C + c] = from_f32<TO>(S * g * sw_sigmoid(g));
    }
    // the last run that holds a token ends at the portion's end: its state is the request's
    const int last = n > 0 ? (n - 1) / per : 0;
    if (n > 0 && warp == last) *slot = S;
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gated_clamp_act_kernel(const TI* __restrict__ gu, const float* __restrict__ dense, TO* __restrict__ out, int N, int E, int ff,
                       int il, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
    const float w = dense != nullptr ? dense[t * E + c / ff] : 1.f;
    float y = 0.f;
    if (w != 0.f) {
      const TI* p = gu + t * 2 * N + (size_t)(c / il) * 2 * il + c % il;
      const float g = fminf(to_f32(p[0]), limit), u = fminf(fmaxf(to_f32(p[il]), -limit), limit);
      y = g * sw_sigmoid(alpha * g) * (u + 1.0f) * w;
    }
    out[t * N + c] = from_f32<TO>(y);
  }
}

// bfloat16 in and out, blocks of 8 (or a multiple): eight columns a thread, one 16-byte load each of gate and up
__global__ void __launch_bounds__(256)
gated_clamp_act_vec_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ dense, __nv_bfloat16* __restrict__ out,
                           int N, int E, int ff, int il, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < N; c += gridDim.y * blockDim.x * 8) {
    const float w = dense != nullptr ? dense[t * E + c / ff] : 1.f;
    uint4 res = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      const __nv_bfloat16* p = gu + t * 2 * N + (size_t)(c / il) * 2 * il + c % il;
      const uint4 graw = *reinterpret_cast<const uint4*>(p), uraw = *reinterpret_cast<const uint4*>(p + il);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
      const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
      __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
        r2[k] = __floats2bfloat162_rn(g.x * sw_sigmoid(alpha * g.x) * (u.x + 1.0f) * w, g.y * sw_sigmoid(alpha * g.y) * (u.y + 1.0f) * w);
      }
    }
    *reinterpret_cast<uint4*>(out + t * N + c) = res;
  }
}

constexpr int RS_WARPS = 4;

// a warp per token
__global__ void __launch_bounds__(RS_WARPS * 32)
moe_route_top_softmax_kernel(const float* __restrict__ logits, int T, int E, int top, float* __restrict__ dense,
                             int* __restrict__ idx, float* __restrict__ wts) {
  extern __shared__ float sm[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * RS_WARPS + warp;
  if (t >= T) return;
  float* choice = sm + (size_t)warp * E;
  const float* z = logits + (size_t)t * E;
  for (int e = lane; e < E; e += 32) {
    choice[e] = z[e];
    dense[(size_t)t * E + e] = 0.f;
  }
  __syncwarp();
  float zmax = 0.f, sum = 0.f;
  for (int n = 0; n < top; ++n) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (!isnan(v) && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int e = bi < E ? bi : 0;
    if (n == 0) zmax = bv;
    const float p = expf(bv - zmax);                 // the winners come in falling order: the first is the largest
    sum += p;
    if (lane == 0) {
      choice[e] = NAN;                                // taken
      idx[(size_t)t * top + n] = e;
      wts[(size_t)t * top + n] = p;
    }
    __syncwarp();
  }
  const float inv = 1.0f / sum;
  if (lane == 0)
    for (int n = 0; n < top; ++n) {
      const float w = wts[(size_t)t * top + n] * inv;
      wts[(size_t)t * top + n] = w;
      dense[(size_t)t * E + idx[(size_t)t * top + n]] = w;
    }
}

// a thread per (token, head, pair or plain column)
template <typename TO>
__global__ void __launch_bounds__(256)
rope_cols_kernel(const float* __restrict__ x, int ldx, int xoff, int xstride, int n, int rot, const int* __restrict__ positions,
                 const float* __restrict__ table, int max_pos, TO* __restrict__ out, int ldo, int ooff, int ostride, int T, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = rot / 2, per = ostride - ooff - half;            // items of a head: pairs first, then single columns and the zero tail
  const size_t total = (size_t)T * H * per;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(e % per);
    const size_t th = e / per;
    const int h = (int)(th % H);
    const size_t t = th / H;
    const float* src = x + t * ldx + xoff + (size_t)h * xstride;
    TO* dst = out + t * ldo + (size_t)h * ostride + ooff;
    if (j < half) {
      int pos = positions[t];
      pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
      const float* cs = table + (size_t)pos * rot;                 // cos[half] then sin[half]
      const float u = src[j], v = src[j + half], c = cs[j], s = cs[half + j];
      dst[j] = from_f32<TO>(u * c - v * s);
      dst[j + half] = from_f32<TO>(v * c + u * s);
    } else {
      const int d = j + half;                                       // a column beyond the rotated ones
      dst[d] = from_f32<TO>(d < n ? src[d] : 0.f);
    }
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_post_add_norm(float* stream_, const float* term, int parts, size_t part_stride, const float* post_gain,
                                   float post_eps, const float* pre_gain, float pre_eps, void* h, int h_dtype, int T, int W,
                                   cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && W > 0, "post_add_norm: bad sizes T=%d W=%d", T, W);
  SLLM_REQUIRE(term == nullptr || (post_gain != nullptr && parts >= 1), "post_add_norm: a term needs its gain");
  SLLM_REQUIRE(h == nullptr || pre_gain != nullptr, "post_add_norm: a normed output needs its gain");
  SLLM_REQUIRE(term != nullptr || h != nullptr, "post_add_norm: nothing to do");
  if (T == 0) return SLLM_OK;
  if (h == nullptr || h_dtype == SLLM_F32)
    launch_kernel(post_add_norm_kernel<float>, (unsigned)T, 256, 0, stream, stream_, term, parts, part_stride, post_gain, post_eps,
                  pre_gain, pre_eps, (float*)h, W);
  else if (h_dtype == SLLM_BF16)
    launch_kernel(post_add_norm_kernel<__nv_bfloat16>, (unsigned)T, 256, 0, stream, stream_, term, parts, part_stride, post_gain,
                  post_eps, pre_gain, pre_eps, (__nv_bfloat16*)h, W);
  else
    SLLM_REQUIRE(false, "post_add_norm: unknown dtype %d", h_dtype);
  return launch_status("post_add_norm");
}

SLLM_EXPORT int sllm_mingru_scan(const float* proj, int ld, int off_z, int off_x, int off_g, float* state, const int* q_start,
                                 const int* state_slots, void* out, int out_dtype, int S, int C, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && C > 0, "mingru_scan: bad sizes S=%d C=%d", S, C);
  SLLM_REQUIRE(off_z >= 0 && off_x >= 0 && off_g >= 0 && off_z + C <= ld && off_x + C <= ld && off_g + C <= ld,
               "mingru_scan: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  const dim3 grid((unsigned)S, (unsigned)((C + 31) / 32));
  SLLM_REQUIRE(grid.y <= 65535, "mingru_scan: %d channels exceed one launch", C);
  if (out_dtype == SLLM_F32)
    launch_kernel(mingru_scan_kernel<float>, grid, 32 * MG_WARPS, 0, stream, proj, ld, off_z, off_x, off_g, state, q_start,
                  state_slots, (float*)out, C);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(mingru_scan_kernel<__nv_bfloat16>, grid, 32 * MG_WARPS, 0, stream, proj, ld, off_z, off_x, off_g, state, q_start,
                  state_slots, (__nv_bfloat16*)out, C);
  else
    SLLM_REQUIRE(false, "mingru_scan: unknown dtype %d", out_dtype);
  return launch_status("mingru_scan");
}

SLLM_EXPORT int sllm_gated_clamp_act(const void* gu, int in_dtype, const float* dense, void* out, int out_dtype, int T, int N, int E,
                                     int ff, int interleave, float limit, float alpha, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && N >= 1 && ff >= 1 && interleave >= 1 && N % interleave == 0, "gated_clamp_act: bad sizes T=%d N=%d ff=%d blocks of %d",
               T, N, ff, interleave);
  SLLM_REQUIRE(dense == nullptr || (E >= 1 && (long)E * ff == N && ff % interleave == 0),
               "gated_clamp_act: %d experts of %d columns in blocks of %d do not make %d", E, ff, interleave, N);
  if (T == 0) return SLLM_OK;
  if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16 && interleave % 8 == 0 && (dense == nullptr || ff % 8 == 0) &&
      (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
    int by = (N / 8 + 255) / 256;
    if (by > 64) by = 64;
    launch_kernel(gated_clamp_act_vec_kernel, dim3((unsigned)T, (unsigned)by), 256, 0, stream, (const __nv_bfloat16*)gu, dense,
                  (__nv_bfloat16*)out, N, E, ff, interleave, limit, alpha);
    return launch_status("gated_clamp_act");
  }
  int by = (N + 255) / 256;
  if (by > 64) by = 64;
  const dim3 grid((unsigned)T, (unsigned)by);
#define LAUNCH(TI, TO) \
  launch_kernel(gated_clamp_act_kernel<TI, TO>, grid, 256, 0, stream, (const TI*)gu, dense, (TO*)out, N, E, ff, interleave, limit, alpha)
  if (in_dtype == SLLM_F32 && out_dtype == SLLM_F32) LAUNCH(float, float);
  else if (in_dtype == SLLM_F32 && out_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "gated_clamp_act: unsupported dtypes %d -> %d", in_dtype, out_dtype);
#undef LAUNCH
  return launch_status("gated_clamp_act");
}

SLLM_EXPORT int sllm_moe_route_top_softmax(const float* logits, int T, int E, int top, float* dense, int* idx, float* wts,
                                           cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && E >= 1 && top >= 1 && top <= E, "moe_route_top_softmax: bad sizes T=%d E=%d top=%d", T, E, top);
  const size_t smem = (size_t)RS_WARPS * E * sizeof(float);
  SLLM_REQUIRE(smem <= 48 * 1024, "moe_route_top_softmax: %d experts are more than the kernel keeps in shared memory", E);
  if (T == 0) return SLLM_OK;
  launch_kernel(moe_route_top_softmax_kernel, (unsigned)((T + RS_WARPS - 1) / RS_WARPS), RS_WARPS * 32, smem, stream, logits, T, E,
                top, dense, idx, wts);
  return launch_status("moe_route_top_softmax");
}

SLLM_EXPORT int sllm_rope_cols(const float* x, int ldx, int xoff, int xstride, int n, int rot, const int* positions,
                               const float* table, int max_pos, void* out, int out_dtype, int ldo, int ooff, int ostride, int T,
                               int H, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && H > 0 && n >= 0 && rot >= 0 && rot % 2 == 0 && rot <= n, "rope_cols: bad sizes T=%d H=%d n=%d rot=%d", T, H, n, rot);
  SLLM_REQUIRE(xoff >= 0 && xstride >= n && xoff + (H - 1) * (long)xstride + n <= ldx, "rope_cols: columns outside the product's %d", ldx);
  SLLM_REQUIRE(ooff >= 0 && ooff + n <= ostride && (long)H * ostride <= ldo, "rope_cols: the slice %d..%d does not fit rows of %d", ooff, ooff + n, ostride);
  SLLM_REQUIRE(rot == 0 || (table != nullptr && max_pos > 0), "rope_cols: rotary table missing");
  const int per = ostride - ooff - rot / 2;
  if (T == 0 || per <= 0) return SLLM_OK;
  const size_t total = (size_t)T * H * per;
  const unsigned blocks = (unsigned)((total + 255) / 256 > 8192 ? 8192 : (total + 255) / 256);
  if (out_dtype == SLLM_F32)
    launch_kernel(rope_cols_kernel<float>, blocks, 256, 0, stream, x, ldx, xoff, xstride, n, rot, positions, table, max_pos,
                  (float*)out, ldo, ooff, ostride, T, H);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(rope_cols_kernel<__nv_bfloat16>, blocks, 256, 0, stream, x, ldx, xoff, xstride, n, rot, positions, table, max_pos,
                  (__nv_bfloat16*)out, ldo, ooff, ostride, T, H);
  else
    SLLM_REQUIRE(false, "rope_cols: unknown dtype %d", out_dtype);
  return launch_status("rope_cols");
}
