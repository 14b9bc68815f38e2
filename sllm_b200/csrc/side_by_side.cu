// Kernels of a layer that runs two mixers side by side: softmax attention with normed queries and keys
// next to a recurrence behind short convolutions, and the normed mean of their outputs.
//
//   qk_norm_rope_kv_write   q | k | v columns of a float32 product: each query and key head over its root mean
//                           square times a gain shared by the heads, then rotated (the first `rot` channels, channel i
//                           with i + rot/2, by the table's cos and sin of the token's position); values as they are.
//                           Queries leave in the compute dtype, keys and values go to their token's place in the pages.
//                           Without gains the heads are not normed; `q_mul` (one number per query head) multiplies the
//                           query head (a factor on its scores).
//                           Key and value sizes may differ: the cache's head is D >= both, the rest is zeros.
//   short_conv_silu         y[t, c] = silu(sum_j w[c, taps-1-j] x[t-j, c]) over a request's own tokens; the taps-1 inputs
//                           before a portion come from the request's state row, zeros before the sequence starts.
//   short_conv_state        the state row receives the portion's last taps-1 inputs (older ones move up).
//   norm_mean_add           stream += (a / rms(a) * ga + b / rms(b) * gb) / 2.
//
// All arithmetic is float32.
#include "common.cuh"

namespace sllm {

__device__ __forceinline__ float sbs_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename TC>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_write_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ q_gain,
                             const float* __restrict__ k_gain, const float* __restrict__ q_mul, float eps,
                             const int* __restrict__ positions,
                             const float* __restrict__ table, int rot, int max_pos, int nq, int nkv, int dim, int vdim, int D,
                             const int* __restrict__ slot_mapping, int page_size, int num_pages, TC* __restrict__ k_cache,
                             TC* __restrict__ v_cache, TC* __restrict__ q_out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)T * heads) return;
  const int t = (int)(item / heads), head = (int)(item % heads);
  const float* row = qkv + (size_t)t * ld;
  TC* dst;
  if (head < nq) {
    dst = q_out + ((size_t)t * nq + head) * D;
  } else {
    if (slot_mapping == nullptr) return;
    const int slot = slot_mapping[t];
    if (slot < 0 || slot / page_size >= num_pages) return;          // a row that writes nothing (padding, a borrowed cache)
    const bool is_k = head < nq + nkv;
    const int kvh = is_k ? head - nq : head - nq - nkv;
    dst = (is_k ? k_cache : v_cache) + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * D;
  }
  if (head >= nq + nkv) {                                            // a value head: copied, zeros beyond vdim
    const float* x = row + (size_t)(nq + nkv) * dim + (size_t)(head - nq - nkv) * vdim;
    for (int d = lane; d < D; d += 32) dst[d] = from_f32<TC>(d < vdim ? x[d] : 0.f);
    return;
  }
  const float* x = row + (size_t)head * dim;
  const float* gain = head < nq ? q_gain : k_gain;
  float inv = 1.0f;
  if (gain != nullptr) {
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) ss = fmaf(x[d], x[d], ss);
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)dim + eps);
  }
  if (head < nq && q_mul != nullptr) inv *= q_mul[head];
  const int half = rot / 2;
  if (rot > 0) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = table + (size_t)pos * rot;                    // cos[half] then sin[half]
    for (int j = lane; j < half; j += 32) {
      const float u = x[j] * inv * (gain ? gain[j] : 1.f), v = x[j + half] * inv * (gain ? gain[j + half] : 1.f);
      const float c = cs[j], sn = cs[half + j];
      dst[j] = from_f32<TC>(u * c - v * sn);
      dst[j + half] = from_f32<TC>(v * c + u * sn);
    }
  }
  for (int d = rot + lane; d < D; d += 32) dst[d] = from_f32<TC>(d < dim ? x[d] * inv * (gain ? gain[d] : 1.f) : 0.f);
}

// grid (T, ceil(C / 256)): a thread per (token, channel).  MODE 0: silu of the convolution; MODE 1: the input plus its
// convolution (a convolution in front of a sublayer that keeps the sublayer's input as it was beside it).
template <int MODE, typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ x, int ld, int off, const float* __restrict__ w, int taps,
                  const float* __restrict__ state, const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                  const int* __restrict__ state_slots, TO* __restrict__ out, int C, int own_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = seq_of_token[t];
  const int first = q_start[seq];
  float* st = const_cast<float*>(state) + ((size_t)state_slots[seq] * C + c) * (taps - 1);
  const float* wc = w + (size_t)c * taps;
  float acc = 0.f, now = 0.f;
  for (int j = taps - 1; j >= 0; --j) {                 // oldest input first: one order whatever the cut
    const int src = t - j;
    const float v = src >= first ? x[(size_t)src * ld + off + c] : st[taps - 1 - (first - src)];
    acc = fmaf(wc[taps - 1 - j], v, acc);
    now = v;
  }
  out[(size_t)t * C + c] = from_f32<TO>(MODE == 0 ? sbs_silu(acc) : now + acc);
  if (own_state) {                                      // every request brings one token: its thread is the state's only reader
    for (int i = 0; i + 1 < taps; ++i) st[i] = i + 2 < taps ? st[i + 1] : now;
  }
}

// The same for four channels a thread (C, ld and off multiples of 4): one 16-byte load per tap of the input, of the
// weights and of the state.  The sums run in the scalar kernel's order, so both give the same bits.
template <int MODE, int TAPS, typename TO>
__global__ void __launch_bounds__(128)
short_conv_vec4_kernel(const float* __restrict__ x, int ld, int off, const float* __restrict__ w, float* __restrict__ state,
                       const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                       TO* __restrict__ out, int C, int own_state) {
  constexpr int KEEP = TAPS - 1;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  const int seq = seq_of_token[t];
  const int first = q_start[seq];
  float wl[4 * TAPS];                                   // [channel][tap]
#pragma unroll
  for (int k = 0; k < TAPS; ++k) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(w + (size_t)c * TAPS) + k);
    wl[4 * k] = q.x; wl[4 * k + 1] = q.y; wl[4 * k + 2] = q.z; wl[4 * k + 3] = q.w;
  }
  float sl[4 * KEEP + 1];                               // [channel][older input], oldest first
  float* sp = state + ((size_t)state_slots[seq] * C + c) * KEEP;
  if (t - first < KEEP) {
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
      const float4 q = *(reinterpret_cast<const float4*>(sp) + k);
      sl[4 * k] = q.x; sl[4 * k + 1] = q.y; sl[4 * k + 2] = q.z; sl[4 * k + 3] = q.w;
    }
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, now[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < TAPS; ++j) {                      // oldest input first
    const int src = t - (KEEP - j);
    if (src >= first) {
      const float4 q = *reinterpret_cast<const float4*>(x + (size_t)src * ld + off + c);
      now[0] = q.x; now[1] = q.y; now[2] = q.z; now[3] = q.w;
    } else {
      const int idx = KEEP - (first - src);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < KEEP; ++k) v = k == idx ? sl[i * KEEP + k] : v;
        now[i] = v;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fmaf(wl[i * TAPS + j], now[i], acc[i]);
  }
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) y[i] = MODE == 0 ? sbs_silu(acc[i]) : now[i] + acc[i];
  if constexpr (sizeof(TO) == 4) {
    *reinterpret_cast<float4*>(out + (size_t)t * C + c) = make_float4(y[0], y[1], y[2], y[3]);
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)t * C + c) = pk;
  }
  if (own_state && KEEP > 0) {                          // one token a request: this thread is the state's only reader
    float nl[4 * KEEP + 1];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int k = 0; k < KEEP; ++k) nl[i * KEEP + k] = k + 1 < KEEP ? sl[i * KEEP + k + 1] : now[i];
#pragma unroll
    for (int k = 0; k < KEEP; ++k)
      *(reinterpret_cast<float4*>(sp) + k) = make_float4(nl[4 * k], nl[4 * k + 1], nl[4 * k + 2], nl[4 * k + 3]);
  }
}

// Long portions: a thread walks RUN consecutive tokens of its four channels with the last inputs in registers, so every
// input row is loaded once instead of once per tap.  Where a run starts, and where the next token belongs to another
// request, the window is read afresh (from the rows before, or from the request's state row).  Sums in the order of the
// kernels above: the same bits.  grid (ceil(T / RUN), ceil(C / 512)).
template <int MODE, int TAPS, typename TO, int RUN>
__global__ void __launch_bounds__(128)
short_conv_run_kernel(const float* __restrict__ x, int ld, int off, const float* __restrict__ w, const float* __restrict__ state,
                      const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                      TO* __restrict__ out, int C, int T) {
  constexpr int KEEP = TAPS - 1;
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * RUN, c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  float wl[4 * TAPS];                                   // [channel][tap]
#pragma unroll
  for (int k = 0; k < TAPS; ++k) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(w + (size_t)c * TAPS) + k);
    wl[4 * k] = q.x; wl[4 * k + 1] = q.y; wl[4 * k + 2] = q.z; wl[4 * k + 3] = q.w;
  }
  float win[KEEP + 1][4];                               // [older input, oldest first][channel]
  float now[4] = {0.f, 0.f, 0.f, 0.f};
  int seq_before = -1;
#pragma unroll
  for (int r = 0; r < RUN; ++r) {
    const int t = t0 + r;
    if (t >= T) break;
    const int seq = seq_of_token[t];
    if (seq != seq_before) {
      const int first = q_start[seq];
      const float* sp = state + ((size_t)state_slots[seq] * C + c) * KEEP;
#pragma unroll
      for (int k = 0; k < KEEP; ++k) {
        const int src = t - KEEP + k;
        if (src >= first) {
          const float4 q = *reinterpret_cast<const float4*>(x + (size_t)src * ld + off + c);
          win[k][0] = q.x; win[k][1] = q.y; win[k][2] = q.z; win[k][3] = q.w;
        } else {
          const int idx = KEEP - (first - src);         // the state row holds the KEEP inputs before `first`
#pragma unroll
          for (int i = 0; i < 4; ++i) win[k][i] = idx >= 0 ? sp[i * KEEP + idx] : 0.f;
        }
      }
      seq_before = seq;
    } else {
#pragma unroll
      for (int k = 0; k + 1 < KEEP; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i) win[k][i] = win[k + 1][i];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (KEEP > 0) win[KEEP - 1][i] = now[i];
    }
    const float4 q = *reinterpret_cast<const float4*>(x + (size_t)t * ld + off + c);
    now[0] = q.x; now[1] = q.y; now[2] = q.z; now[3] = q.w;
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < KEEP; ++k) acc = fmaf(wl[i * TAPS + k], win[k][i], acc);
      acc = fmaf(wl[i * TAPS + KEEP], now[i], acc);
      y[i] = MODE == 0 ? sbs_silu(acc) : now[i] + acc;
    }
    if constexpr (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(out + (size_t)t * C + c) = make_float4(y[0], y[1], y[2], y[3]);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(out + (size_t)t * C + c) = pk;
    }
  }
}

// grid (S, ceil(C / 256)): a thread per (request, channel) rewrites its state row in ascending order
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const float* __restrict__ x, int ld, int off, int taps, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ state_slots, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int first = q_start[seq], n = q_start[seq + 1] - first, keep = taps - 1;
  float* st = state + ((size_t)state_slots[seq] * C + c) * keep;
  for (int i = 0; i < keep; ++i) {
    const int idx = n - keep + i;                       // which of the portion's tokens, negative: still the old state's
    st[i] = idx >= 0 ? x[(size_t)(first + idx) * ld + off + c] : st[i + n];
  }
}

// a CTA per token
__global__ void __launch_bounds__(256)
norm_mean_add_kernel(float* __restrict__ stream, const float* __restrict__ a, const float* __restrict__ ga,
                     const float* __restrict__ b, const float* __restrict__ gb, float eps, int W) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * W;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float va = a[base + i], vb = b[base + i];
    sa = fmaf(va, va, sa);
    sb = fmaf(vb, vb, sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ia = 1.0f / sqrtf(sa / (float)W + eps), ib = 1.0f / sqrtf(sb / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    stream[base + i] += 0.5f * (a[base + i] * ia * ga[i] + b[base + i] * ib * gb[i]);
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_qk_norm_rope_kv_write(const float* qkv, int ld, const float* q_gain, const float* k_gain, const float* q_mul, float eps,
                                           const int* positions, const float* table, int rot, int max_pos, int nq, int nkv,
                                           int dim, int vdim, int D, const int* slot_mapping, int page_size, int num_pages,
                                           void* k_cache, void* v_cache, void* q_out, int cache_dtype, int T, cudaStream_t stream) {
  SLLM_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "qk_norm_rope: query and key heads are normed together or not at all");
  SLLM_REQUIRE(T >= 0 && nq > 0 && nkv > 0 && dim > 0 && vdim > 0, "qk_norm_rope: bad sizes T=%d nq=%d nkv=%d dim=%d vdim=%d", T, nq, nkv, dim, vdim);
  SLLM_REQUIRE(D >= dim && D >= vdim, "qk_norm_rope: the cache's head of %d is smaller than a key of %d or a value of %d", D, dim, vdim);
  SLLM_REQUIRE(ld >= (nq + nkv) * dim + nkv * vdim, "qk_norm_rope: the product's %d columns are fewer than q|k|v", ld);
  SLLM_REQUIRE(rot >= 0 && rot <= dim && rot % 2 == 0, "qk_norm_rope: rotary_dim=%d must be even and <= %d", rot, dim);
  SLLM_REQUIRE(rot == 0 || (table != nullptr && max_pos > 0), "qk_norm_rope: rotary table missing");
  SLLM_REQUIRE(slot_mapping == nullptr || (page_size > 0 && num_pages > 0 && k_cache && v_cache), "qk_norm_rope: cache arguments missing");
  if (T == 0) return SLLM_OK;
  const long items = (long)T * (nq + 2 * nkv);
  const unsigned blocks = (unsigned)((items + 3) / 4);
#define LAUNCH(TC)                                                                                                        \
  launch_kernel(qk_norm_rope_kv_write_kernel<TC>, blocks, 128, 0, stream, qkv, ld, q_gain, k_gain, q_mul, eps, positions, table, rot, \
                max_pos, nq, nkv, dim, vdim, D, slot_mapping, page_size, num_pages, (TC*)k_cache, (TC*)v_cache, (TC*)q_out, T)
  if (cache_dtype == SLLM_F32) LAUNCH(float);
  else if (cache_dtype == SLLM_BF16) LAUNCH(__nv_bfloat16);
  else SLLM_REQUIRE(false, "qk_norm_rope: unknown dtype %d", cache_dtype);
#undef LAUNCH
  return launch_status("qk_norm_rope_kv_write");
}

// mode 0: silu(conv(x)), float32 out; mode 1: x + conv(x) in `out_dtype`.  The state rows are rewritten by a second launch,
// or, where every request brings one token, by the threads that read them.
SLLM_EXPORT int sllm_short_conv(const float* x, int ld, int off, const float* w, int taps, float* state, const int* seq_of_token,
                                const int* q_start, const int* state_slots, void* out, int out_dtype, int mode, int T, int S, int C,
                                cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && S >= 0 && C > 0 && taps >= 1 && off >= 0 && off + C <= ld, "short_conv: bad sizes T=%d C=%d taps=%d", T, C, taps);
  SLLM_REQUIRE(taps == 1 || state != nullptr, "short_conv: a convolution over %d taps needs its state", taps);
  SLLM_REQUIRE((mode == 0 && out_dtype == SLLM_F32) || (mode == 1 && (out_dtype == SLLM_F32 || out_dtype == SLLM_BF16)),
               "short_conv: mode %d with output dtype %d", mode, out_dtype);
  if (T == 0) return SLLM_OK;
  const unsigned cb = (unsigned)((C + 255) / 256);
  const dim3 grid((unsigned)T, cb);
  // as many tokens as requests: each brings one, and the thread that reads a state row may rewrite it (one launch)
  const int own_state = (T == S && taps > 1) ? 1 : 0;
  const bool vec = taps >= 2 && taps <= 4 && C % 4 == 0 && ld % 4 == 0 && off % 4 == 0 && (uintptr_t)x % 16 == 0 &&
                   (uintptr_t)w % 16 == 0 && (uintptr_t)state % 16 == 0 && (uintptr_t)out % 16 == 0;
  constexpr int CONV_RUN = 8;
  if (vec && !own_state && T >= CONV_RUN * S) {         // portions of eight tokens and more on average
    const dim3 rgrid((unsigned)((T + CONV_RUN - 1) / CONV_RUN), (unsigned)((C / 4 + 127) / 128));
#define RUNK(MODE_, TAPS_, TO_)                                                                                            \
  launch_kernel(short_conv_run_kernel<MODE_, TAPS_, TO_, CONV_RUN>, rgrid, 128, 0, stream, x, ld, off, w, (const float*)state, \
                seq_of_token, q_start, state_slots, (TO_*)out, C, T)
#define RUN_TAPS(MODE_, TO_)                          \
  if (taps == 2) RUNK(MODE_, 2, TO_);                 \
  else if (taps == 3) RUNK(MODE_, 3, TO_);            \
  else RUNK(MODE_, 4, TO_)
    if (mode == 0) { RUN_TAPS(0, float); }
    else if (out_dtype == SLLM_F32) { RUN_TAPS(1, float); }
    else { RUN_TAPS(1, __nv_bfloat16); }
#undef RUN_TAPS
#undef RUNK
  } else if (vec) {
    const dim3 vgrid((unsigned)T, (unsigned)((C / 4 + 127) / 128));
#define VEC(MODE_, TAPS_, TO_)                                                                                              \
  launch_kernel(short_conv_vec4_kernel<MODE_, TAPS_, TO_>, vgrid, 128, 0, stream, x, ld, off, w, state, seq_of_token, q_start, \
                state_slots, (TO_*)out, C, own_state)
#define VEC_TAPS(MODE_, TO_)                          \
  if (taps == 2) VEC(MODE_, 2, TO_);                  \
  else if (taps == 3) VEC(MODE_, 3, TO_);             \
  else VEC(MODE_, 4, TO_)
    if (mode == 0) { VEC_TAPS(0, float); }
    else if (out_dtype == SLLM_F32) { VEC_TAPS(1, float); }
    else { VEC_TAPS(1, __nv_bfloat16); }
#undef VEC_TAPS
#undef VEC
  } else if (mode == 0)
    launch_kernel(short_conv_kernel<0, float>, grid, 256, 0, stream, x, ld, off, w, taps, (const float*)state, seq_of_token, q_start,
                  state_slots, (float*)out, C, own_state);
  else if (out_dtype == SLLM_F32)
    launch_kernel(short_conv_kernel<1, float>, grid, 256, 0, stream, x, ld, off, w, taps, (const float*)state, seq_of_token, q_start,
                  state_slots, (float*)out, C, own_state);
  else
    launch_kernel(short_conv_kernel<1, __nv_bfloat16>, grid, 256, 0, stream, x, ld, off, w, taps, (const float*)state, seq_of_token,
                  q_start, state_slots, (__nv_bfloat16*)out, C, own_state);
  int rc = launch_status("short_conv");
  if (rc != SLLM_OK || taps == 1 || S == 0 || own_state) return rc;
  launch_kernel(short_conv_state_kernel, dim3((unsigned)S, cb), 256, 0, stream, x, ld, off, taps, state, q_start, state_slots, C);
  return launch_status("short_conv_state");
}

SLLM_EXPORT int sllm_short_conv_silu(const float* x, int ld, int off, const float* w, int taps, float* state,
                                     const int* seq_of_token, const int* q_start, const int* state_slots, float* out, int T,
                                     int S, int C, cudaStream_t stream) {
  return sllm_short_conv(x, ld, off, w, taps, state, seq_of_token, q_start, state_slots, out, SLLM_F32, 0, T, S, C, stream);
}

SLLM_EXPORT int sllm_norm_mean_add(float* stream_, const float* a, const float* ga, const float* b, const float* gb, float eps,
                                   int T, int W, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && W > 0, "norm_mean_add: bad sizes T=%d W=%d", T, W);
  if (T == 0) return SLLM_OK;
  launch_kernel(norm_mean_add_kernel, (unsigned)T, 256, 0, stream, stream_, a, ga, b, gb, eps, W);
  return launch_status("norm_mean_add");
}
