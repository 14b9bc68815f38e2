// Kernels of latent attention: every head's keys and values are up-projections of one small latent
// vector per token, and only that vector is cached.
//
//   * latent_write: the latent of each new token (columns of a float32 product) over its root mean square,
//     times a gain, written to the token's place in the paged cache in the cache's dtype.
//   * head_linear: a product per head, out[t, h, :] = W_h x[t, h, :], with W [H, dout, din].  It carries a
//     head's query into the latent space (W_h = the head's key up-projection, transposed: the score of a
//     query against a key is then its carried form against the cached latent) and the head's weighted sum
//     of latents back out through the value up-projection; there the result can be multiplied by
//     sigmoid(gate[t, h]) as it is written.  float32 accumulation over din in a fixed order: on the CUDA cores
//     for the float32 path, on the tensor cores (mma.sync) for bfloat16 operands.
#include "common.cuh"
#include "mma.cuh"

namespace sllm {

// With `tail` > 0 the `tail` columns after the latent are one more key part that every head shares: not normed, its first
// `rot` channels rotated by position (rotate-half layout), written behind the latent; rows of the cache are D wide,
// zeros beyond rank + tail.
template <typename TC>
__global__ void latent_write_kernel(const float* __restrict__ proj, int ld, int off, int rank, const float* __restrict__ gain,
                                    float eps, const int* __restrict__ slot_mapping, TC* __restrict__ cache, int D, int tail,
                                    int rot, const int* __restrict__ positions, const float* __restrict__ table, int max_pos) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  const float* x = proj + (size_t)t * ld + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
  const float total = block_sum(ss, red);
  if (slot < 0) return;               // a row that pads the batch: no place to write to
  const float inv = 1.0f / sqrtf(total / (float)rank + eps);
  TC* dst = cache + (size_t)slot * D;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<TC>(x[i] * inv * gain[i]);
  const float* y = x + rank;
  const int half = rot / 2;
  if (half > 0) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = table + (size_t)pos * rot;                    // cos[half] then sin[half]
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const float u = y[j], v = y[j + half], c = cs[j], sn = cs[half + j];
      dst[rank + j] = from_f32<TC>(u * c - v * sn);
      dst[rank + j + half] = from_f32<TC>(v * c + u * sn);
    }
  }
  for (int d = rank + rot + threadIdx.x; d < D; d += blockDim.x) dst[d] = from_f32<TC>(d < rank + tail ? y[d - rank] : 0.f);
}

constexpr int HL_BM = 64, HL_BN = 64, HL_BK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_linear_kernel(const TX* __restrict__ x, int ldx, int xoff, const TW* __restrict__ w, TO* __restrict__ out,
                   const float* __restrict__ gate, int ldg, int goff, int T, int H, int din, int dout, int xstride, int ldo,
                   int ostride, int gate_elem) {
  __shared__ float Xs[HL_BK][HL_BM + 4];
  __shared__ float Ws[HL_BK][HL_BN + 4];
  pdl_wait();
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int lr = tid / 4, lk = (tid % 4) * 4;
  const TX* xh = x + xoff + (size_t)h * xstride;
  const TW* wh = w + (size_t)h * dout * din;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < din; k0 += HL_BK) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gk = k0 + lk + i;
      a[i] = (m0 + lr < T && gk < din) ? to_f32(xh[(size_t)(m0 + lr) * ldx + gk]) : 0.f;
      b[i] = (n0 + lr < dout && gk < din) ? to_f32(wh[(size_t)(n0 + lr) * din + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) { Xs[lk + i][lr] = a[i]; Ws[lk + i][lr] = b[i]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HL_BK; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= T) continue;
    const float g = (gate != nullptr && !gate_elem) ? 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + goff + h])) : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= dout) continue;
      const float ge = (gate != nullptr && gate_elem) ? 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + goff + (size_t)h * dout + n])) : g;
      out[(size_t)m * ldo + (size_t)h * ostride + n] = from_f32<TO>(acc[i][j] * ge);
    }
  }
}

// The same product on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation) for the
// bfloat16 path: a CTA of four warps makes 64 tokens x 64 outputs of one head, a warp 16 tokens x 64; x (bfloat16, or
// float32 rounded to bfloat16 as it is staged) and W_h are staged 32 columns of din at a time in shared memory,
// rows padded to 40 elements so that the fragments' 32-bit reads fall in distinct banks.
constexpr int HM_BM = 64, HM_BN = 64, HM_BK = 32, HM_LD = HM_BK + 8;

template <typename TX>
__global__ void __launch_bounds__(128)
head_linear_mma_kernel(const TX* __restrict__ x, int ldx, int xoff, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ out, const float* __restrict__ gate, int ldg, int goff, int T, int H,
                       int din, int dout, int vec, int xstride, int ldo, int ostride, int gate_elem) {
  __shared__ __align__(16) __nv_bfloat16 Xs[HM_BM][HM_LD];
  __shared__ __align__(16) __nv_bfloat16 Ws[HM_BN][HM_LD];
  pdl_wait();
  const int h = blockIdx.z, m0 = blockIdx.y * HM_BM, n0 = blockIdx.x * HM_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
  const TX* xh = x + xoff + (size_t)h * xstride;
  const __nv_bfloat16* wh = w + (size_t)h * dout * din;
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
  for (int k0 = 0; k0 < din; k0 += HM_BK) {
    __syncthreads();
    // stage x: 64 rows x 32 columns
    if (vec) {
      if constexpr (sizeof(TX) == 2) {
        for (int c = tid; c < HM_BM * 4; c += 128) {
          const int r = c >> 2, kc = (c & 3) * 8;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (m0 + r < T && k0 + kc < din) v = *reinterpret_cast<const uint4*>(xh + (size_t)(m0 + r) * ldx + k0 + kc);
          *reinterpret_cast<uint4*>(&Xs[r][kc]) = v;
        }
      } else {
        for (int c = tid; c < HM_BM * 8; c += 128) {
          const int r = c >> 3, kc = (c & 7) * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (m0 + r < T && k0 + kc < din) v = *reinterpret_cast<const float4*>(xh + (size_t)(m0 + r) * ldx + k0 + kc);
          *reinterpret_cast<uint2*>(&Xs[r][kc]) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
        }
      }
      for (int c = tid; c < HM_BN * 4; c += 128) {
        const int r = c >> 2, kc = (c & 3) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n0 + r < dout && k0 + kc < din) v = *reinterpret_cast<const uint4*>(wh + (size_t)(n0 + r) * din + k0 + kc);
        *reinterpret_cast<uint4*>(&Ws[r][kc]) = v;
      }
    } else {
      for (int c = tid; c < HM_BM * HM_BK; c += 128) {
        const int r = c / HM_BK, k = c % HM_BK;
        Xs[r][k] = (m0 + r < T && k0 + k < din) ? from_f32<__nv_bfloat16>(to_f32(xh[(size_t)(m0 + r) * ldx + k0 + k])) : __float2bfloat16_rn(0.f);
        Ws[r][k] = (n0 + r < dout && k0 + k < din) ? wh[(size_t)(n0 + r) * din + k0 + k] : __float2bfloat16_rn(0.f);
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HM_BK; kk += 16) {
      unsigned a[4];
      const int r = warp * 16 + g;
      a[0] = *reinterpret_cast<const unsigned*>(&Xs[r][kk + 2 * t4]);
      a[1] = *reinterpret_cast<const unsigned*>(&Xs[r + 8][kk + 2 * t4]);
      a[2] = *reinterpret_cast<const unsigned*>(&Xs[r][kk + 8 + 2 * t4]);
      a[3] = *reinterpret_cast<const unsigned*>(&Xs[r + 8][kk + 8 + 2 * t4]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned b0 = *reinterpret_cast<const unsigned*>(&Ws[j * 8 + g][kk + 2 * t4]);
        const unsigned b1 = *reinterpret_cast<const unsigned*>(&Ws[j * 8 + g][kk + 8 + 2 * t4]);
        mma_bf16(acc[j], a, b0, b1);
      }
    }
  }
  pdl_launch_dependents();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int m = m0 + warp * 16 + g + half * 8;
    if (m >= T) continue;
    const float gt = (gate != nullptr && !gate_elem) ? 1.0f / (1.0f + expf(-gate[(size_t)m * ldg + goff + h])) : 1.0f;
    const float* ge = (gate != nullptr && gate_elem) ? gate + (size_t)m * ldg + goff + (size_t)h * dout : nullptr;
    __nv_bfloat16* o = out + (size_t)m * ldo + (size_t)h * ostride;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j * 8 + 2 * t4;
      if (n < dout) o[n] = __float2bfloat16_rn(acc[j][half * 2] * (ge ? 1.0f / (1.0f + expf(-ge[n])) : gt));
      if (n + 1 < dout) o[n + 1] = __float2bfloat16_rn(acc[j][half * 2 + 1] * (ge ? 1.0f / (1.0f + expf(-ge[n + 1])) : gt));
    }
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_latent_rope_write(const float* proj, int ld, int off, int rank, int tail, int rot, const float* gain, float eps,
                                       const int* positions, const float* table, int max_pos, const int* slot_mapping, void* cache,
                                       int cache_dtype, int D, int T, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && rank > 0 && tail >= 0 && off >= 0 && off + rank + tail <= ld, "latent_write: columns %d..%d of %d", off,
               off + rank + tail, ld);
  SLLM_REQUIRE(D >= rank + tail, "latent_write: rows of %d do not hold %d + %d", D, rank, tail);
  SLLM_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= tail, "latent_write: %d rotated channels of %d", rot, tail);
  SLLM_REQUIRE(rot == 0 || (positions != nullptr && table != nullptr && max_pos > 0), "latent_write: rotary table missing");
  if (T == 0) return SLLM_OK;
  const int threads = rank >= 512 ? 256 : 128;
  if (cache_dtype == SLLM_F32)
    launch_kernel(latent_write_kernel<float>, T, threads, 0, stream, proj, ld, off, rank, gain, eps, slot_mapping, (float*)cache, D,
                  tail, rot, positions, table, max_pos);
  else if (cache_dtype == SLLM_BF16)
    launch_kernel(latent_write_kernel<__nv_bfloat16>, T, threads, 0, stream, proj, ld, off, rank, gain, eps, slot_mapping,
                  (__nv_bfloat16*)cache, D, tail, rot, positions, table, max_pos);
  else
    SLLM_REQUIRE(false, "latent_write: unknown dtype %d", cache_dtype);
  return launch_status("latent_write");
}

SLLM_EXPORT int sllm_latent_write(const float* proj, int ld, int off, int rank, const float* gain, float eps,
                                  const int* slot_mapping, void* cache, int cache_dtype, int T, cudaStream_t stream) {
  return sllm_latent_rope_write(proj, ld, off, rank, 0, 0, gain, eps, nullptr, nullptr, 0, slot_mapping, cache, cache_dtype, rank, T,
                                stream);
}

// Heads `xstride` apart in x (>= din) and `ostride` apart in rows of `ldo` of the output (>= dout; what lies between is
// left as it is).  gate_elem 0: one gate logit per (token, head); 1: one per output element, at goff + h*dout + n.
SLLM_EXPORT int sllm_head_linear_strided(const void* x, int x_dtype, int ldx, int xoff, int xstride, const void* w, int w_dtype,
                                         void* out, int out_dtype, int ldo, int ostride, const float* gate, int ldg, int goff,
                                         int gate_elem, int T, int H, int din, int dout, cudaStream_t stream) {
  SLLM_REQUIRE(T >= 0 && H > 0 && H <= 65535 && din > 0 && dout > 0, "head_linear: bad sizes T=%d H=%d din=%d dout=%d", T, H, din, dout);
  SLLM_REQUIRE(xstride >= din && xoff >= 0 && xoff + (long)(H - 1) * xstride + din <= ldx, "head_linear: columns %d.. of %d", xoff, ldx);
  SLLM_REQUIRE(ostride >= dout && (long)(H - 1) * ostride + dout <= ldo, "head_linear: %d heads of %d do not fit rows of %d", H, ostride, ldo);
  SLLM_REQUIRE(gate == nullptr || (goff >= 0 && goff + (gate_elem ? (long)H * dout : (long)H) <= ldg), "head_linear: gate columns outside %d", ldg);
  if (T == 0) return SLLM_OK;
  const dim3 grid((unsigned)((dout + HL_BN - 1) / HL_BN), (unsigned)((T + HL_BM - 1) / HL_BM), (unsigned)H);
  SLLM_REQUIRE(grid.y <= 65535, "head_linear: too many rows for one launch");
#define SLLM_HL(TX, TW, TO)                                                                                              \
  launch_kernel(head_linear_kernel<TX, TW, TO>, grid, 256, 0, stream, (const TX*)x, ldx, xoff, (const TW*)w, (TO*)out, gate, ldg, \
                goff, T, H, din, dout, xstride, ldo, ostride, gate_elem)
  if (w_dtype == SLLM_BF16 && out_dtype == SLLM_BF16 && (x_dtype == SLLM_F32 || x_dtype == SLLM_BF16)) {
    // the bfloat16 path: tensor cores; 16-byte loads where every row of x and of W starts on a 16-byte boundary
    const int xe = x_dtype == SLLM_F32 ? 4 : 8;
    const int vec = din % 8 == 0 && ldx % xe == 0 && xoff % xe == 0 && xstride % xe == 0 && ((uintptr_t)x & 15) == 0 &&
                    ((uintptr_t)w & 15) == 0;
    if (x_dtype == SLLM_F32)
      launch_kernel(head_linear_mma_kernel<float>, grid, 128, 0, stream, (const float*)x, ldx, xoff, (const __nv_bfloat16*)w,
                    (__nv_bfloat16*)out, gate, ldg, goff, T, H, din, dout, vec, xstride, ldo, ostride, gate_elem);
    else
      launch_kernel(head_linear_mma_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, ldx, xoff,
                    (const __nv_bfloat16*)w, (__nv_bfloat16*)out, gate, ldg, goff, T, H, din, dout, vec, xstride, ldo, ostride, gate_elem);
    return launch_status("head_linear");
  }
  if (x_dtype == SLLM_F32 && w_dtype == SLLM_F32 && out_dtype == SLLM_F32) SLLM_HL(float, float, float);
  else SLLM_REQUIRE(false, "head_linear: dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
#undef SLLM_HL
  return launch_status("head_linear");
}

SLLM_EXPORT int sllm_head_linear(const void* x, int x_dtype, int ldx, int xoff, const void* w, int w_dtype, void* out, int out_dtype,
                                 const float* gate, int ldg, int goff, int T, int H, int din, int dout, cudaStream_t stream) {
  return sllm_head_linear_strided(x, x_dtype, ldx, xoff, din, w, w_dtype, out, out_dtype, H * dout, dout, gate, ldg, goff, 0, T, H, din,
                                  dout, stream);
}
