// Kernels of layers that wrap each sublayer in two norms, and of the small recurrent and gated units such layers hold.
//
//   * post_add_norm: a sublayer's output is normed BEFORE it joins the stream, and the stream is normed for the next
//     reader in the same pass:  stream += term / rms(term) * post_gain;  h = stream / rms(stream) * pre_gain.  Either
//     half may be absent (the first norm of a model has no term; the last sublayer has no reader).  A CTA per token,
//     float32 throughout; `term` may be a stack of k-split partial sums.  post_add_norm_conv: where every request
//     brings one token, the reader's input convolution rides along: h + conv(h) from the request's state row, which the
//     same thread then rewrites (the sums in the convolution kernel's order, oldest input first).
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

// stream += term / rms(term) * post_gain (no term: nothing added); returns this thread's share of sum(stream^2)
__device__ __forceinline__ float post_add(float* __restrict__ x, const float* __restrict__ term, size_t base, int parts,
                                          size_t part_stride, const float* __restrict__ post_gain, float post_eps, int W, float* red) {
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
  return ss;
}

// The same with the row in registers (W <= 256 * PER): the stream's and the term's loads leave together, nothing is read
// twice, and the sums run in the order of `post_add`, so both forms give the same bits.
template <int PER>
__device__ __forceinline__ float post_add_regs(float* __restrict__ x, const float* __restrict__ term, size_t base, int parts,
                                               size_t part_stride, const float* __restrict__ post_gain, float post_eps, int W,
                                               float* red, float (&y)[PER]) {
  float v[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int i = threadIdx.x + k * 256;
    y[k] = i < W ? x[i] : 0.f;
  }
  float ss = 0.f;
  if (term != nullptr) {
    float st = 0.f;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
      float t = 0.f;
      if (i < W) {
        t = term[base + i];
        for (int p = 1; p < parts; ++p) t += term[p * part_stride + base + i];
        st = fmaf(t, t, st);
      }
      v[k] = t;
    }
    st = block_sum(st, red);
    const float inv = 1.0f / sqrtf(st / (float)W + post_eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < W) {
        y[k] = y[k] + v[k] * inv * post_gain[i];
        x[i] = y[k];
        ss = fmaf(y[k], y[k], ss);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < PER; ++k)
      if ((int)threadIdx.x + k * 256 < W) ss = fmaf(y[k], y[k], ss);
  }
  return ss;
}

// PER = 0: rows of any width, read from memory in every pass
template <typename TO, int PER>
__global__ void __launch_bounds__(256)
post_add_norm_kernel(float* __restrict__ stream, const float* __restrict__ term, int parts, size_t part_stride,
                     const float* __restrict__ post_gain, float post_eps, const float* __restrict__ pre_gain, float pre_eps,
                     TO* __restrict__ h, int W) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float* x = stream + base;
  if constexpr (PER > 0) {
    float y[PER];
    float ss = post_add_regs<PER>(x, term, base, parts, part_stride, post_gain, post_eps, W, red, y);
    if (h == nullptr) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < W) h[base + i] = from_f32<TO>(y[k] * inv * pre_gain[i]);
    }
  } else {
    float ss = post_add(x, term, base, parts, part_stride, post_gain, post_eps, W, red);
    if (h == nullptr) return;
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) h[base + i] = from_f32<TO>(x[i] * inv * pre_gain[i]);
  }
}

// h + conv(h) of one channel from its state row (oldest input first), which moves on by one
template <typename TO>
__device__ __forceinline__ void conv_one(float now, const float* __restrict__ w, float* __restrict__ s, int keep, TO* __restrict__ dst) {
  float acc = 0.f;
  for (int j = 0; j < keep; ++j) {
    const float v = s[j];
    acc = fmaf(w[j], v, acc);
    if (j > 0) s[j - 1] = v;
  }
  acc = fmaf(w[keep], now, acc);
  if (keep > 0) s[keep - 1] = now;
  *dst = from_f32<TO>(now + acc);
}

// A CTA per token, every token its request's only one in the step: the normed row h never leaves the CTA; out = h + conv(h)
// with the request's earlier inputs from its state row [W, taps-1] (oldest first), which moves on by one.  TAPS > 0 (with
// PER > 0): the taps are known when compiling, and all of a thread's state rows and weights are loaded before the first
// store, so the loads of its channels do not wait for one another.
template <typename TO, int PER, int TAPS>
__global__ void __launch_bounds__(256)
post_add_norm_conv_kernel(float* __restrict__ stream, const float* __restrict__ term, int parts, size_t part_stride,
                          const float* __restrict__ post_gain, float post_eps, const float* __restrict__ pre_gain, float pre_eps,
                          const float* __restrict__ conv_w, int taps, float* __restrict__ conv_state,
                          const int* __restrict__ seq_of_token, const int* __restrict__ state_slots, TO* __restrict__ out, int W) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float* x = stream + base;
  const int keep = taps - 1;
  float* st = keep > 0 ? conv_state + (size_t)state_slots[seq_of_token[blockIdx.x]] * W * keep : nullptr;
  if constexpr (PER > 0 && TAPS > 0) {
    constexpr int KEEP = TAPS - 1;
    float sv[PER][KEEP + 1], wv[PER][TAPS], pg[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
#pragma unroll
      for (int j = 0; j < KEEP; ++j) sv[k][j] = i < W ? st[(size_t)i * KEEP + j] : 0.f;
#pragma unroll
      for (int j = 0; j < TAPS; ++j) wv[k][j] = i < W ? conv_w[(size_t)i * TAPS + j] : 0.f;
      pg[k] = i < W ? pre_gain[i] : 0.f;
    }
    float y[PER];
    float ss = post_add_regs<PER>(x, term, base, parts, part_stride, post_gain, post_eps, W, red, y);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < W) {
        const float now = y[k] * inv * pg[k];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {                  // oldest input first
          acc = fmaf(wv[k][j], sv[k][j], acc);
          if (j > 0) st[(size_t)i * KEEP + j - 1] = sv[k][j];
        }
        acc = fmaf(wv[k][KEEP], now, acc);
        if (KEEP > 0) st[(size_t)i * KEEP + KEEP - 1] = now;
        out[base + i] = from_f32<TO>(now + acc);
      }
    }
  } else if constexpr (PER > 0) {
    float y[PER];
    float ss = post_add_regs<PER>(x, term, base, parts, part_stride, post_gain, post_eps, W, red, y);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < W) conv_one(y[k] * inv * pre_gain[i], conv_w + (size_t)i * taps, st + (size_t)i * keep, keep, out + base + i);
    }
  } else {
    float ss = post_add(x, term, base, parts, part_stride, post_gain, post_eps, W, red);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)W + pre_eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x)
      conv_one(x[i] * inv * pre_gain[i], conv_w + (size_t)i * taps, st + (size_t)i * keep, keep, out + base + i);
  }
}

constexpr int MG_WARPS = 16;

// grid (S, ceil(C / CH)), 32 * MG_WARPS threads.  A warp holds CH channels (its lanes' low bits) and 32 / CH runs of tokens:
// CH = 32 where requests bring few tokens (a warp a run, 128-byte rows), CH = 8 for long portions (four times the CTAs and
// the runs, 32-byte rows).  A run's effect on what it meets is (keep, reach): S_out = keep * S_in + reach.
template <typename TO, int CH>
__global__ void __launch_bounds__(32 * MG_WARPS)
mingru_scan_kernel(const float* __restrict__ proj, int ld, int off_z, int off_x, int off_g, float* __restrict__ state,
                   const int* __restrict__ q_start, const int* __restrict__ state_slots, TO* __restrict__ out, int C) {
  constexpr int RUNS = MG_WARPS * (32 / CH);
  __shared__ float keep_s[RUNS][CH], reach_s[RUNS][CH];
  pdl_wait();
  const int seq = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ch = lane % CH, run = warp * (32 / CH) + lane / CH;
  const int c = blockIdx.y * CH + ch;
  const bool live = c < C;
  const int first = q_start[seq], n = q_start[seq + 1] - first;
  const int per = (n + RUNS - 1) / RUNS;
  const int lo = min(n, run * per), hi = min(n, lo + per);
  float* slot = state + (size_t)state_slots[seq] * C + c;
  float S = live ? *slot : 0.f;                  // read before the barrier: the last run's thread writes it at its end
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
  keep_s[run][ch] = keep;
  reach_s[run][ch] = reach;
  __syncthreads();
  for (int w = 0; w < run; ++w) S = fmaf(keep_s[w][ch], S, reach_s[w][ch]);           // this run's entry state
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
    if (n > 0 && run == last) *slot = S;
  }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gated_clamp_act_kernel(const TI* __restrict__ gu, const float* __restrict__ dense, TO* __restrict__ out, int N, int E, int ff,
                       int il, float limit, float alpha, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
    const float w = dense != nullptr ? dense[t * E + c / ff] : 1.f;
    float y = 0.f;
    if (w != 0.f) {
      const TI* p = gu + t * 2 * N + (size_t)(c / il) * 2 * il + c % il;
      if (act == 1) {                              // silu(g) * u
        const float g = to_f32(p[0]);
        y = g * sw_sigmoid(g) * to_f32(p[il]) * w;
      } else {
        const float g = fminf(to_f32(p[0]), limit), u = fminf(fmaxf(to_f32(p[il]), -limit), limit);
        y = g * sw_sigmoid(alpha * g) * (u + 1.0f) * w;
      }
    }
    out[t * N + c] = from_f32<TO>(y);
  }
}

// bfloat16 in and out, blocks of 8 (or a multiple): eight columns a thread, one 16-byte load each of gate and up
__global__ void __launch_bounds__(256)
gated_clamp_act_vec_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ dense, __nv_bfloat16* __restrict__ out,
                           int N, int E, int ff, int il, float limit, float alpha, int act) {
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
        if (act == 1) {
          r2[k] = __floats2bfloat162_rn(g.x * sw_sigmoid(g.x) * u.x * w, g.y * sw_sigmoid(g.y) * u.y * w);
          continue;
        }
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
moe_route_top_softmax_kernel(const float* __restrict__ logits, int T, int E, int top, float scale, float* __restrict__ dense,
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
  const float inv = scale / sum;
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
#define PAN(TO_, PER_)                                                                                                      \
  launch_kernel(post_add_norm_kernel<TO_, PER_>, (unsigned)T, 256, 0, stream, stream_, term, parts, part_stride, post_gain, \
                post_eps, pre_gain, pre_eps, (TO_*)h, W)
#define PAN_W(TO_)                       \
  if (W <= 1024) PAN(TO_, 4);            \
  else if (W <= 2048) PAN(TO_, 8);       \
  else if (W <= 4096) PAN(TO_, 16);      \
  else PAN(TO_, 0)
  if (h == nullptr || h_dtype == SLLM_F32) { PAN_W(float); }
  else if (h_dtype == SLLM_BF16) { PAN_W(__nv_bfloat16); }
  else
    SLLM_REQUIRE(false, "post_add_norm: unknown dtype %d", h_dtype);
#undef PAN_W
#undef PAN
  return launch_status("post_add_norm");
}

SLLM_EXPORT int sllm_post_add_norm_conv(float* stream_, const float* term, int parts, size_t part_stride, const float* post_gain,
                                        float post_eps, const float* pre_gain, float pre_eps, const float* conv_w, int taps,
                                        float* conv_state, const int* seq_of_token, const int* state_slots, void* out, int out_dtype,
                                        int T, int W, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && W > 0 && taps >= 1, "post_add_norm_conv: bad sizes T=%d W=%d taps=%d", T, W, taps);
  SLLM_REQUIRE(term == nullptr || (post_gain != nullptr && parts >= 1), "post_add_norm_conv: a term needs its gain");
  SLLM_REQUIRE(pre_gain != nullptr && conv_w != nullptr && out != nullptr, "post_add_norm_conv: the norm's gain, the taps and an output");
  SLLM_REQUIRE(taps == 1 || conv_state != nullptr, "post_add_norm_conv: %d taps need the requests' state rows", taps);
  if (T == 0) return SLLM_OK;
#define PANC(TO_, PER_, TAPS_)                                                                                               \
  launch_kernel(post_add_norm_conv_kernel<TO_, PER_, TAPS_>, (unsigned)T, 256, 0, stream, stream_, term, parts, part_stride, \
                post_gain, post_eps, pre_gain, pre_eps, conv_w, taps, conv_state, seq_of_token, state_slots, (TO_*)out, W)
#define PANC_T(TO_, PER_)                  \
  if (taps == 2) PANC(TO_, PER_, 2);       \
  else if (taps == 3) PANC(TO_, PER_, 3);  \
  else if (taps == 4) PANC(TO_, PER_, 4);  \
  else PANC(TO_, PER_, 0)
#define PANC_W(TO_)                                 \
  if (W <= 1024) { PANC_T(TO_, 4); }                \
  else if (W <= 2048) { PANC_T(TO_, 8); }           \
  else if (W <= 4096) { PANC_T(TO_, 16); }          \
  else PANC(TO_, 0, 0)
  if (out_dtype == SLLM_F32) { PANC_W(float); }
  else if (out_dtype == SLLM_BF16) { PANC_W(__nv_bfloat16); }
  else
    SLLM_REQUIRE(false, "post_add_norm_conv: unknown dtype %d", out_dtype);
#undef PANC_W
#undef PANC_T
#undef PANC
  return launch_status("post_add_norm_conv");
}

SLLM_EXPORT int sllm_mingru_scan(const float* proj, int ld, int off_z, int off_x, int off_g, float* state, const int* q_start,
                                 const int* state_slots, void* out, int out_dtype, int T, int S, int C, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && T >= 0 && C > 0, "mingru_scan: bad sizes T=%d S=%d C=%d", T, S, C);
  SLLM_REQUIRE(off_z >= 0 && off_x >= 0 && off_g >= 0 && off_z + C <= ld && off_x + C <= ld && off_g + C <= ld,
               "mingru_scan: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  // long portions (a request's share of the step's tokens: 256 and more): many short runs of few channels
  const bool narrow = T / S >= 256;
  const int ch = narrow ? 8 : 32;
  const dim3 grid((unsigned)S, (unsigned)((C + ch - 1) / ch));
  SLLM_REQUIRE(grid.y <= 65535, "mingru_scan: %d channels exceed one launch", C);
#define MG(TO_, CH_)                                                                                                         \
  launch_kernel(mingru_scan_kernel<TO_, CH_>, grid, 32 * MG_WARPS, 0, stream, proj, ld, off_z, off_x, off_g, state, q_start, \
                state_slots, (TO_*)out, C)
  if (out_dtype == SLLM_F32) {
    if (narrow) MG(float, 8); else MG(float, 32);
  } else if (out_dtype == SLLM_BF16) {
    if (narrow) MG(__nv_bfloat16, 8); else MG(__nv_bfloat16, 32);
  } else
    SLLM_REQUIRE(false, "mingru_scan: unknown dtype %d", out_dtype);
#undef MG
  return launch_status("mingru_scan");
}

SLLM_EXPORT int sllm_gated_clamp_act(const void* gu, int in_dtype, const float* dense, void* out, int out_dtype, int T, int N, int E,
                                     int ff, int interleave, float limit, float alpha, int act, cudaStream_t stream) {
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
                  (__nv_bfloat16*)out, N, E, ff, interleave, limit, alpha, act);
    return launch_status("gated_clamp_act");
  }
  int by = (N + 255) / 256;
  if (by > 64) by = 64;
  const dim3 grid((unsigned)T, (unsigned)by);
#define LAUNCH(TI, TO) \
  launch_kernel(gated_clamp_act_kernel<TI, TO>, grid, 256, 0, stream, (const TI*)gu, dense, (TO*)out, N, E, ff, interleave, limit, alpha, act)
  if (in_dtype == SLLM_F32 && out_dtype == SLLM_F32) LAUNCH(float, float);
  else if (in_dtype == SLLM_F32 && out_dtype == SLLM_BF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "gated_clamp_act: unsupported dtypes %d -> %d", in_dtype, out_dtype);
#undef LAUNCH
  return launch_status("gated_clamp_act");
}

SLLM_EXPORT int sllm_moe_route_top_softmax(const float* logits, int T, int E, int top, float scale, float* dense, int* idx, float* wts,
                                           cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && E >= 1 && top >= 1 && top <= E, "moe_route_top_softmax: bad sizes T=%d E=%d top=%d", T, E, top);
  const size_t smem = (size_t)RS_WARPS * E * sizeof(float);
  SLLM_REQUIRE(smem <= 48 * 1024, "moe_route_top_softmax: %d experts are more than the kernel keeps in shared memory", E);
  if (T == 0) return SLLM_OK;
  launch_kernel(moe_route_top_softmax_kernel, (unsigned)((T + RS_WARPS - 1) / RS_WARPS), RS_WARPS * 32, smem, stream, logits, T, E,
                top, scale, dense, idx, wts);
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
