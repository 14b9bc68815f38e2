// Memory-bound kernels of a "parallel" block (one norm whose output both the mixer and the feed-forward
// read) and of an input with sinusoidal positions:
//   * a sinusoidal position vector added to the float32 stream;
//   * the pending terms added into the stream and, per row and group, 1/sqrt(mean square + eps) of the
//     stream (an RMS norm taken over `groups` equal consecutive parts of the vector);
//   * that norm applied (times a gain), with an optional token shift: the mixer's input is the row blended
//     with the previous token's normed row, which for the first token of a portion comes from the
//     request's state slot; the slot then receives the portion's last normed row;
//   * act(gate) * up of a gate|up product, act = SiLU or the tanh form of GELU;
//   * an activation over some columns of a float32 product.
// All arithmetic in float32; the stream, the gains, the state and the reciprocal roots are float32.
#include "common.cuh"

namespace sllm {

// stream[t, 2i] += sin(p * f_i), stream[t, 2i+1] += cos(p * f_i), p = positions[t], f = inv_freq[i].
// The angle is a float32 product of the float32 position and the float32 frequency; sinf and cosf are
// the accurate forms (their argument reduction is exact for angles of this size).
__global__ void add_sinusoid_kernel(float* __restrict__ stream, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  float* row = stream + (size_t)t * W;
  for (int i = threadIdx.x; i < W / 2; i += blockDim.x) {
    const float ang = p * inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    row[2 * i] += s;
    row[2 * i + 1] += c;
  }
}

__device__ __forceinline__ float4 pb_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 pb_load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void pb_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void pb_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&a);
  raw.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// Row t of the stream takes the pending terms (each a stack of `parts` partial sums, float32); then, if
// rinv is given, rinv[t, g] = 1 / sqrt(mean(stream[t, group g]^2) + eps).  A warp owns a group (warps take
// groups in turn) and sums it in an order that depends on the group's size only.  VEC: W and the stacks'
// strides are multiples of 4 and every pointer is 16-byte aligned; four elements a thread, the partial sums
// read with independent loads.
template <bool VEC>
__global__ void add_group_ssq_kernel(float* __restrict__ stream, const float* __restrict__ d0, int parts0, size_t stride0,
                                     const float* __restrict__ d1, int parts1, size_t stride1,
                                     float* __restrict__ rinv, int W, int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  float* row = stream + (size_t)t * W;
  if (d0 != nullptr || d1 != nullptr) {
    if constexpr (VEC) {
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
        float4 v = pb_load4(row + i);
        if (d0 != nullptr) {
#pragma unroll 8
          for (int p = 0; p < parts0; ++p) {
            const float4 x = pb_load4(d0 + p * stride0 + (size_t)t * W + i);
            v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
          }
        }
        if (d1 != nullptr) {
#pragma unroll 8
          for (int p = 0; p < parts1; ++p) {
            const float4 x = pb_load4(d1 + p * stride1 + (size_t)t * W + i);
            v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
          }
        }
        pb_store4(row + i, v);
      }
    } else {
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float v = row[i];
        if (d0 != nullptr)
          for (int p = 0; p < parts0; ++p) v += d0[p * stride0 + (size_t)t * W + i];
        if (d1 != nullptr)
          for (int p = 0; p < parts1; ++p) v += d1[p * stride1 + (size_t)t * W + i];
        row[i] = v;
      }
    }
    __syncthreads();       // the block's own writes are read back below
  }
  if (rinv == nullptr) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int gs = W / groups;
  for (int g = warp; g < groups; g += nw) {
    const float* x = row + (size_t)g * gs;
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) rinv[(size_t)t * groups + g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
}

// 1 / sqrt(mean(x[group]^2) + eps) of every group of a row, into dst[groups] (shared memory): warps take groups in
// turn; a group's sum is taken in an order that depends on its size only.
template <bool VEC>
__device__ __forceinline__ void group_roots(const float* __restrict__ row, float* dst, int groups, int gs, float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nw) {
    const float* x = row + (size_t)g * gs;
    float ss = 0.f;
    if constexpr (VEC) {
      for (int i = lane * 4; i < gs; i += 128) {
        const float4 v = pb_load4(x + i);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
    } else {
      for (int i = lane; i < gs; i += 32) ss = fmaf(x[i], x[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) dst[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
}

// h[t, i] = stream[t, i] * rinv[t, g(i)] * gain[i]                      -> out_h (if given)
// hs[t, i] = h + (h_prev - h) * mix[i]                                   -> out_hs (if mix is given)
// h_prev is the normed row t-1 of the same request's portion, or state[slot] for the portion's first
// token; the block of that first token then writes the portion's last normed row to state[slot] (each
// thread reads its channels of the slot before it writes them; no other block touches the slot).
// rinv == nullptr: the block takes the reciprocal roots of the rows it reads itself (the row, and the row
// before or the portion's last), so that a stream with nothing pending needs no kernel before this one.
// VEC: W and W / groups are multiples of 4 and every pointer is 16-byte aligned.
template <typename TO, bool VEC>
__global__ void group_norm_shift_kernel(const float* __restrict__ stream, const float* __restrict__ rinv,
                                        const float* __restrict__ gain, const float* __restrict__ mix,
                                        float* __restrict__ state, const int* __restrict__ seq_of_token,
                                        const int* __restrict__ q_start, const int* __restrict__ state_slots,
                                        TO* __restrict__ out_h, TO* __restrict__ out_hs, int W, int groups, float eps) {
  extern __shared__ float s_ri[];          // [2][groups]: this row's roots, and the other row's
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int gs = W / groups;
  const float* row = stream + (size_t)t * W;
  int first_t = t, last_t = t;
  bool first = false;
  float* slot = nullptr;
  if (mix != nullptr) {
    const int s = seq_of_token[t];
    first_t = q_start[s];
    last_t = q_start[s + 1] - 1;
    first = t == first_t;
    slot = state + (size_t)state_slots[s] * W;
  }
  // the other row: the one before (its normed form is h_prev), or for a portion's first token the portion's last
  const int other_t = mix == nullptr ? t : (first ? last_t : t - 1);
  const float* orow = stream + (size_t)other_t * W;
  const float* ri;
  const float* ori;
  if (rinv != nullptr) {
    ri = rinv + (size_t)t * groups;
    ori = rinv + (size_t)other_t * groups;
  } else {
    group_roots<VEC>(row, s_ri, groups, gs, eps);
    if (other_t != t) group_roots<VEC>(orow, s_ri + groups, groups, gs, eps);
    __syncthreads();
    ri = s_ri;
    ori = other_t != t ? s_ri + groups : s_ri;
  }
  if constexpr (VEC) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      const int g = i / gs;
      const float4 x = pb_load4(row + i), w = pb_load4(gain + i);
      const float r = ri[g];
      const float4 h = make_float4(x.x * r * w.x, x.y * r * w.y, x.z * r * w.z, x.w * r * w.w);
      if (out_h != nullptr) pb_store4(out_h + (size_t)t * W + i, h);
      if (mix == nullptr) continue;
      const float4 ox = pb_load4(orow + i);
      const float orr = ori[g];
      const float4 oh = make_float4(ox.x * orr * w.x, ox.y * orr * w.y, ox.z * orr * w.z, ox.w * orr * w.w);
      float4 hp = oh;
      if (first) {
        hp = pb_load4(slot + i);
        pb_store4(slot + i, oh);
      }
      const float4 m = pb_load4(mix + i);
      pb_store4(out_hs + (size_t)t * W + i, make_float4(h.x + (hp.x - h.x) * m.x, h.y + (hp.y - h.y) * m.y,
                                                        h.z + (hp.z - h.z) * m.z, h.w + (hp.w - h.w) * m.w));
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const int g = i / gs;
      const float w = gain[i];
      const float h = row[i] * ri[g] * w;
      if (out_h != nullptr) out_h[(size_t)t * W + i] = from_f32<TO>(h);
      if (mix == nullptr) continue;
      const float oh = orow[i] * ori[g] * w;
      float hp = oh;
      if (first) {
        hp = slot[i];
        slot[i] = oh;
      }
      out_hs[(size_t)t * W + i] = from_f32<TO>(h + (hp - h) * mix[i]);
    }
  }
}

__device__ __forceinline__ float act_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float act_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[t, i] = act(gate) * up; gate and up alternate along a row of gu in blocks of `interleave` columns
// (interleave == I: all gates, then all ups).  VEC: I and interleave are multiples of 4 and the pointers 16-byte
// aligned; four results a thread.
template <typename TI, typename TO, int ACT, bool VEC>
__global__ void act_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int I, int interleave) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;             // (rows on the grid's x: no limit of 65,535)
  constexpr int PER = VEC ? 4 : 1;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * PER; i < I; i += gridDim.y * blockDim.x * PER) {
    const int b = i / interleave, o = i % interleave;
    const TI* p = gu + t * 2 * I + (size_t)b * 2 * interleave + o;
    if constexpr (VEC) {
      const float4 g = pb_load4(p), u = pb_load4(p + interleave);
      float4 r;
      r.x = (ACT == 0 ? act_silu(g.x) : act_gelu_tanh(g.x)) * u.x;
      r.y = (ACT == 0 ? act_silu(g.y) : act_gelu_tanh(g.y)) * u.y;
      r.z = (ACT == 0 ? act_silu(g.z) : act_gelu_tanh(g.z)) * u.z;
      r.w = (ACT == 0 ? act_silu(g.w) : act_gelu_tanh(g.w)) * u.w;
      pb_store4(out + t * I + i, r);
    } else {
      const float g = to_f32(p[0]), u = to_f32(p[interleave]);
      out[t * I + i] = from_f32<TO>((ACT == 0 ? act_silu(g) : act_gelu_tanh(g)) * u);
    }
  }
}

// out[t, j] = tanh(x[t, col0 + j]), j < n; x float32 with row stride ld.
template <typename TO>
__global__ void tanh_cols_kernel(const float* __restrict__ x, int ld, int col0, int n, TO* __restrict__ out, int T) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)T * n;
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t t = e / n;
    const int j = (int)(e % n);
    out[e] = from_f32<TO>(tanhf(x[t * ld + col0 + j]));
  }
}

// stream[t, c] += rows[t, c] + vec[c] (rows may be absent): what a range of layers that runs again takes in before a pass.
__global__ void __launch_bounds__(256)
add_rows_kernel(float* __restrict__ stream, const float* __restrict__ rows, const float* __restrict__ vec, size_t n, int W) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = stream[i];
    if (rows != nullptr) v += rows[i];
    if (vec != nullptr) v += vec[i % W];
    stream[i] = v;
  }
}

// Two norms of one row: out_a = x / sqrt(mean(x^2) + eps) * gain_a and out_b likewise with gain_b (out_b may be absent).
// A CTA per row; the row's sum of squares is taken once, in an order that depends on the width alone.
template <typename TO>
__global__ void __launch_bounds__(256)
norm_pair_kernel(const float* __restrict__ stream, const float* __restrict__ gain_a, const float* __restrict__ gain_b, float eps,
                 TO* __restrict__ out_a, TO* __restrict__ out_b, int W) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const float* x = stream + (size_t)blockIdx.x * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(x[c], x[c], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = x[c] * inv;
    out_a[(size_t)blockIdx.x * W + c] = from_f32<TO>(v * gain_a[c]);
    if (out_b != nullptr) out_b[(size_t)blockIdx.x * W + c] = from_f32<TO>(v * gain_b[c]);
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_add_sinusoid(float* stream, const int* positions, const float* inv_freq, int T, int W,
                                  cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && W > 0 && W % 2 == 0, "add_sinusoid: the width %d must be even", W);
  if (T == 0) return SLLM_OK;
  launch_kernel(add_sinusoid_kernel, T, W >= 2048 ? 256 : 128, 0, stream_, stream, positions, inv_freq, W);
  return launch_status("add_sinusoid");
}

SLLM_EXPORT int sllm_add_group_ssq(float* stream, const float* d0, int parts0, size_t stride0, const float* d1, int parts1,
                                   size_t stride1, float* rinv, int T, int W, int groups, float eps, cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && W > 0 && groups > 0 && W % groups == 0, "add_group_ssq: %d groups do not divide the width %d", groups, W);
  SLLM_REQUIRE((d0 == nullptr || parts0 >= 1) && (d1 == nullptr || parts1 >= 1), "add_group_ssq: bad parts");
  if (T == 0) return SLLM_OK;
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = W % 4 == 0 && stride0 % 4 == 0 && stride1 % 4 == 0 && aligned(stream) && aligned(d0) && aligned(d1);
  const int threads = W >= 4096 ? 256 : 128;
  if (vec) launch_kernel(add_group_ssq_kernel<true>, T, threads, 0, stream_, stream, d0, parts0, stride0, d1, parts1, stride1, rinv, W, groups, eps);
  else launch_kernel(add_group_ssq_kernel<false>, T, threads, 0, stream_, stream, d0, parts0, stride0, d1, parts1, stride1, rinv, W, groups, eps);
  return launch_status("add_group_ssq");
}

SLLM_EXPORT int sllm_group_norm_shift(const float* stream, const float* rinv, const float* gain, const float* mix, float* state,
                                      const int* seq_of_token, const int* q_start, const int* state_slots, void* out_h,
                                      void* out_hs, int out_dtype, int T, int W, int groups, float eps, cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && W > 0 && groups > 0 && W % groups == 0, "group_norm_shift: %d groups do not divide the width %d", groups, W);
  SLLM_REQUIRE(mix != nullptr ? (state && seq_of_token && q_start && state_slots && out_hs) : (out_h != nullptr),
               "group_norm_shift: a shift needs its state, the batch's description and an output; a plain norm needs an output");
  SLLM_REQUIRE(groups <= 4096, "group_norm_shift: %d groups", groups);
  if (T == 0) return SLLM_OK;
  const int threads = W >= 2048 ? 256 : 128;
  const size_t smem = 2 * (size_t)groups * sizeof(float);
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = W % 4 == 0 && (W / groups) % 4 == 0 && aligned(stream) && aligned(gain) && aligned(mix) && aligned(state) &&
                   aligned(out_h) && aligned(out_hs);
#define SLLM_GNS(TO, VEC_)                                                                                                 \
  launch_kernel(group_norm_shift_kernel<TO, VEC_>, T, threads, smem, stream_, stream, rinv, gain, mix, state, seq_of_token, \
                q_start, state_slots, (TO*)out_h, (TO*)out_hs, W, groups, eps)
  if (out_dtype == SLLM_F32) { if (vec) SLLM_GNS(float, true); else SLLM_GNS(float, false); }
  else if (out_dtype == SLLM_BF16) { if (vec) SLLM_GNS(__nv_bfloat16, true); else SLLM_GNS(__nv_bfloat16, false); }
  else SLLM_REQUIRE(false, "group_norm_shift: unknown dtype %d", out_dtype);
#undef SLLM_GNS
  return launch_status("group_norm_shift");
}

SLLM_EXPORT int sllm_act_mul(const void* gu, int in_dtype, void* out, int out_dtype, int T, int I, int interleave, int act,
                             cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && I > 0 && interleave > 0 && I % interleave == 0, "act_mul: bad sizes T=%d I=%d interleave=%d", T, I, interleave);
  SLLM_REQUIRE(act == 0 || act == 1, "act_mul: activation %d is neither 0 (silu) nor 1 (gelu_tanh)", act);
  if (T == 0) return SLLM_OK;
  const int per_block = 256 * 4;
  const dim3 grid((unsigned)T, (unsigned)((I + per_block - 1) / per_block > 64 ? 64 : (I + per_block - 1) / per_block));
  const bool vec = I % 4 == 0 && interleave % 4 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0;
#define SLLM_ACT_MUL(TI, TO)                                                                                                       \
  do {                                                                                                                             \
    if (act == 0 && vec) launch_kernel(act_mul_kernel<TI, TO, 0, true>, grid, 256, 0, stream_, (const TI*)gu, (TO*)out, I, interleave);  \
    else if (act == 0) launch_kernel(act_mul_kernel<TI, TO, 0, false>, grid, 256, 0, stream_, (const TI*)gu, (TO*)out, I, interleave);  \
    else if (vec) launch_kernel(act_mul_kernel<TI, TO, 1, true>, grid, 256, 0, stream_, (const TI*)gu, (TO*)out, I, interleave);   \
    else launch_kernel(act_mul_kernel<TI, TO, 1, false>, grid, 256, 0, stream_, (const TI*)gu, (TO*)out, I, interleave);           \
  } while (0)
  if (in_dtype == SLLM_F32 && out_dtype == SLLM_F32) SLLM_ACT_MUL(float, float);
  else if (in_dtype == SLLM_F32 && out_dtype == SLLM_BF16) SLLM_ACT_MUL(float, __nv_bfloat16);
  else if (in_dtype == SLLM_BF16 && out_dtype == SLLM_BF16) SLLM_ACT_MUL(__nv_bfloat16, __nv_bfloat16);
  else SLLM_REQUIRE(false, "act_mul: dtypes %d -> %d", in_dtype, out_dtype);
#undef SLLM_ACT_MUL
  return launch_status("act_mul");
}

SLLM_EXPORT int sllm_tanh_cols(const float* x, int ld, int col0, int n, void* out, int out_dtype, int T, cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && n > 0 && col0 >= 0 && col0 + n <= ld, "tanh_cols: columns %d..%d of %d", col0, col0 + n, ld);
  if (T == 0) return SLLM_OK;
  const size_t total = (size_t)T * n;
  const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
  if (out_dtype == SLLM_F32) launch_kernel(tanh_cols_kernel<float>, blocks, 256, 0, stream_, x, ld, col0, n, (float*)out, T);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(tanh_cols_kernel<__nv_bfloat16>, blocks, 256, 0, stream_, x, ld, col0, n, (__nv_bfloat16*)out, T);
  else SLLM_REQUIRE(false, "tanh_cols: unknown dtype %d", out_dtype);
  return launch_status("tanh_cols");
}

SLLM_EXPORT int sllm_add_rows(float* stream, const float* rows, const float* vec, int T, int W, cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && W > 0, "add_rows: bad sizes T=%d W=%d", T, W);
  if (T == 0) return SLLM_OK;
  const size_t n = (size_t)T * W;
  size_t blocks = (n + 1023) / 1024;
  if (blocks > 4096) blocks = 4096;
  launch_kernel(add_rows_kernel, (unsigned)blocks, 256, 0, stream_, stream, rows, vec, n, W);
  return launch_status("add_rows");
}

SLLM_EXPORT int sllm_norm_pair(const float* stream, const float* gain_a, const float* gain_b, float eps, void* out_a, void* out_b,
                               int out_dtype, int T, int W, cudaStream_t stream_) {
  SLLM_REQUIRE(T >= 0 && W > 0 && gain_a && out_a && ((gain_b == nullptr) == (out_b == nullptr)), "norm_pair: bad arguments T=%d W=%d", T, W);
  if (T == 0) return SLLM_OK;
  const int threads = W >= 2048 ? 256 : 128;
  if (out_dtype == SLLM_F32)
    launch_kernel(norm_pair_kernel<float>, T, threads, 0, stream_, stream, gain_a, gain_b, eps, (float*)out_a, (float*)out_b, W);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(norm_pair_kernel<__nv_bfloat16>, T, threads, 0, stream_, stream, gain_a, gain_b, eps, (__nv_bfloat16*)out_a,
                  (__nv_bfloat16*)out_b, W);
  else
    SLLM_REQUIRE(false, "norm_pair: unknown dtype %d", out_dtype);
  return launch_status("norm_pair");
}
