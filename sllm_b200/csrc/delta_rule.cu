// The generalized delta rule: a recurrent mixer with a float32 matrix state S [dk, dv] per request and head.
//
//   S <- diag(d) S - (a * u) (u^T S) + k v^T        (S on the right is the state before the token)
//   o  = S^T r
//
// d = exp(-exp(-1/2) * sigmoid(decay logit)) per key channel, a = sigmoid(removal logit + bias) per key
// channel, u = k / sqrt(sum(k^2) + 1e-6) per head.  Everything that enters the recurrence is float32: the
// projections arrive as float32 columns of one product, the decays, rates, unit keys, the state and the
// outputs are float32.
//
// The columns of S evolve independently of one another (column j needs u, d, a*u, k, r of the token and
// v_j only), so a CTA owns a slice of 16 CB columns of one (request, head) and walks the request's tokens in
// order.  Eight consecutive lanes share CB columns, each lane holding every eighth row of them in registers; the
// two sums over rows of a step end in shuffles among the eight.  CB = 4 (a token's five vectors are read from
// shared memory once per four columns: a quarter of the shared-memory reads and of the CTAs) when the batch has
// enough (request, head) pairs to fill the device; CB = 1 when it has not: four times the CTAs, a quarter of the
// work per lane and token, so that one long prompt's walk is as short as it gets.  Four warps compute; four more prepare the next chunk of tokens in the
// other half of shared memory meanwhile (unit keys, decays, rates: a warp per token, all of a token's loads in
// flight at once), so the walk never waits for global memory: one CTA-wide barrier per chunk, none per token.
// A portion of a prompt and a single decoded token run through the same kernel, from the state slot and back
// into it.
//
// Two more recurrences walk the same way, because each is the line above with other vectors in the five places
// (`mode`; only what the loader warps prepare differs):
//   the gated delta rule (mode 1):  S <- g S;  w = beta (v - S^T k^);  S <- S + k^ w^T;  o = S^T q^
//       with k^ = k / sqrt(sum(k^2) + 1e-6), q^ likewise times r_scale, beta = sigmoid(b), g = exp(-exp(A) softplus(a + dt))
//       one number per head.  In terms of the state before the token: S <- g S - (beta g k^)(k^^T S) + k^ (beta v)^T,
//       so u = k = k^, d = g on every row, a*u = beta g k^, v = beta v, r = q^; the walk's own form for this mode reads
//       the key once and the head's two numbers g and beta g: S <- g S + k^ (beta v - beta g (k^^T S))^T.  Several value
//       heads may share one query/key head (head h reads key head h / hdiv).
//   gated linear attention (mode 2):  S <- diag(alpha) S + k v^T;  o = S^T (q r_scale),  alpha = sigmoid(z)^(1/tau) per key
//       channel: u = a*u = 0, d = alpha; the walk's form for this mode has no sum before the update.
//   linear attention with one fixed decay per head (mode 3):  S <- decay_h S + k v^T;  o = S^T q  with q, k and v each
//       through silu first: mode 2's walk with d = decay_h on every row.
//   linear attention whose forget gate also writes (mode 4):  S <- diag(f) S + (1 - f) v^T;  o = S^T silu(q)  with
//       f = lower + (1 - lower) sigmoid(z + bias) per key channel: mode 2's walk with d = f and k = 1 - f.
//
// A second kernel finishes the mixer's output: each head's o over its root mean square, times a gain,
// times sigmoid(gate logit), in the compute dtype.
#include "common.cuh"

namespace sllm {

constexpr int DR_COMPUTE = 128;   // threads that walk the tokens (as many again prepare the next chunk)
constexpr int DR_THREADS = 2 * DR_COMPUTE;
constexpr int DR_MAX_CHUNK = 16;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

struct DeltaParams {
  const float* proj;       // [T, ld]: columns off_r, off_k (+ h*dk), off_v (+ h*dv), off_a (+ h*dk)
  const float* decay;      // [T, H*dk] decay logits
  const float* a_bias;     // [H*dk]
  float* state;            // [slots, H, dk, dv]
  const int* q_start;      // [S+1]
  const int* state_slots;  // [S]
  float* out;              // [T, H*dv]
  int ld, off_r, off_k, off_v, off_a, H, dk, dv, chunk, max_q;
  // modes 1 and 2 (see the head of the file)
  int mode, hdiv;          // hdiv: value heads per query/key head
  const float* gates;      // mode 1: [T, ldg] with beta logits at off_b + h and decay logits at off_dt + h
  int ldg, off_b, off_dt;
  const float* a_log;      // mode 1: [H]
  const float* dt_bias;    // mode 1: [H]
  float r_scale, inv_tau;  // the read-out's factor; mode 2: 1 / tau
};

// RPT: rows of a column per lane (dk <= 8 * RPT = DKP, the padded key size).
constexpr int DR_SPLIT = 8;

template <int RPT, int CB>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(const DeltaParams p) {
  constexpr int SPLIT = DR_SPLIT, COLS = DR_COMPUTE / SPLIT * CB, DKP = RPT * SPLIT, PER_LANE = (DKP + 31) / 32;
  constexpr int VPL = (COLS + 31) / 32;       // values of v a loader lane brings
  extern __shared__ __align__(16) float sm[];
  const int dk = p.dk, dv = p.dv, chunk = p.chunk;
  const int buf_floats = chunk * (5 * DKP + COLS);
  pdl_wait();
  const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * COLS;
  const int t_begin = p.q_start[seq], t_end = p.q_start[seq + 1];
  const int tid = threadIdx.x, lane = tid & 31;
  const bool loader = tid >= DR_COMPUTE;
  const int nchunks = (t_end - t_begin + chunk - 1) / chunk;

  // a loader warp prepares token after token of chunk c: rows of u, d, a*u, k, r (zeros beyond dk) and v's slice
  auto prepare = [&](int c) {
    float* b = sm + (c & 1) * buf_floats;
    float* s_u = b, *s_d = b + chunk * DKP, *s_au = b + 2 * chunk * DKP, *s_k = b + 3 * chunk * DKP, *s_r = b + 4 * chunk * DKP;
    float* s_v = b + 5 * chunk * DKP;
    const int t0 = t_begin + c * chunk, nt = min(chunk, t_end - t0);
    const float c_decay = -expf(-0.5f);
    constexpr int TPW = DR_MAX_CHUNK / (DR_COMPUTE / 32);       // tokens of a chunk per loader warp
    const int lw = (tid - DR_COMPUTE) >> 5;
    float k[TPW][PER_LANE], a[TPW][PER_LANE], d[TPW][PER_LANE], r[TPW][PER_LANE], v[TPW][VPL];
    // every load of the warp's tokens first, then the arithmetic: the loads of all of them are in flight together
#pragma unroll
    for (int q = 0; q < TPW; ++q) {
      const int tt = lw + q * (DR_COMPUTE / 32);
      const bool tok = tt < nt;
      const float* row = p.proj + (size_t)(t0 + (tok ? tt : 0)) * p.ld;
      const float* dec = p.decay + (size_t)(t0 + (tok ? tt : 0)) * p.H * dk + h * dk;
      const int kh = h / p.hdiv;
#pragma unroll
      for (int m = 0; m < PER_LANE; ++m) {
        const int i = lane + 32 * m;
        const bool in = tok && i < dk;
        k[q][m] = in ? __ldg(row + p.off_k + kh * dk + i) : 0.f;
        a[q][m] = (in && p.mode == 0) ? __ldg(row + p.off_a + h * dk + i) + __ldg(p.a_bias + h * dk + i) : 0.f;
        if (p.mode == 4) a[q][m] = in ? __ldg(p.a_bias + h * dk + i) : 0.f;        // the gate's bias; k holds its logit
        d[q][m] = (in && (p.mode == 0 || p.mode == 2)) ? __ldg(dec + i) : 0.f;
        r[q][m] = in ? __ldg(row + p.off_r + kh * dk + i) : 0.f;
      }
#pragma unroll
      for (int m = 0; m < VPL; ++m) {
        const int j = c0 + lane + 32 * m;
        v[q][m] = (tok && lane + 32 * m < COLS && j < dv) ? __ldg(row + p.off_v + h * dv + j) : 0.f;
      }
    }
#pragma unroll
    for (int q = 0; q < TPW; ++q) {
      const int tt = lw + q * (DR_COMPUTE / 32);
      if (tt >= nt) break;
      float ss = 0.f;
#pragma unroll
      for (int m = 0; m < PER_LANE; ++m) ss = fmaf(k[q][m], k[q][m], ss);
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + 1e-6f);
      float vmul = 1.f;
      if (p.mode == 0) {
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) {
          const int i = lane + 32 * m;
          if (i < DKP) {
            const bool in = i < dk;
            const float u = k[q][m] * inv;
            s_k[tt * DKP + i] = k[q][m];
            s_u[tt * DKP + i] = u;
            s_au[tt * DKP + i] = in ? sigmoidf_(a[q][m]) * u : 0.f;
            s_d[tt * DKP + i] = in ? expf(c_decay * sigmoidf_(d[q][m])) : 0.f;
            s_r[tt * DKP + i] = r[q][m];
          }
        }
      } else if (p.mode == 1) {
        float sr = 0.f;
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) sr = fmaf(r[q][m], r[q][m], sr);
        sr = warp_sum(sr);
        const float rinv = p.r_scale / sqrtf(sr + 1e-6f);
        const float* gr = p.gates + (size_t)(t0 + tt) * p.ldg;
        const float beta = sigmoidf_(__ldg(gr + p.off_b + h));
        const float x = __ldg(gr + p.off_dt + h) + __ldg(p.dt_bias + h);
        const float g = expf(-expf(__ldg(p.a_log + h)) * (fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)))));
        vmul = beta;
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) {
          const int i = lane + 32 * m;
          if (i < DKP) {
            s_k[tt * DKP + i] = k[q][m] * inv;
            s_r[tt * DKP + i] = r[q][m] * rinv;
          }
        }
        if (lane == 0) {              // the walk reads the head's two numbers from here (see its mode 1)
          s_u[tt * DKP] = g;
          s_u[tt * DKP + 1] = beta * g;
        }
      } else if (p.mode == 3) {
        const float dh = __ldg(p.a_log + h);           // the head's fixed decay
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) {
          const int i = lane + 32 * m;
          if (i < DKP) {
            s_k[tt * DKP + i] = k[q][m] * sigmoidf_(k[q][m]);
            s_d[tt * DKP + i] = i < dk ? dh : 0.f;
            s_r[tt * DKP + i] = r[q][m] * sigmoidf_(r[q][m]);
          }
        }
#pragma unroll
        for (int m = 0; m < VPL; ++m) v[q][m] *= sigmoidf_(v[q][m]);
      } else if (p.mode == 4) {
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) {
          const int i = lane + 32 * m;
          if (i < DKP) {
            const bool in = i < dk;
            const float lo = in ? __ldg(p.a_log + h * dk + i) : 0.f;                 // the gate's lower bound
            const float f = lo + (1.0f - lo) * sigmoidf_(k[q][m] + a[q][m]);
            s_k[tt * DKP + i] = in ? 1.0f - f : 0.f;
            s_d[tt * DKP + i] = in ? f : 0.f;
            s_r[tt * DKP + i] = r[q][m] * sigmoidf_(r[q][m]);
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < PER_LANE; ++m) {
          const int i = lane + 32 * m;
          if (i < DKP) {
            const bool in = i < dk;
            const float z = d[q][m];
            s_k[tt * DKP + i] = k[q][m];
            s_d[tt * DKP + i] = in ? expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * p.inv_tau) : 0.f;
            s_r[tt * DKP + i] = r[q][m] * p.r_scale;
          }
        }
      }
#pragma unroll
      for (int m = 0; m < VPL; ++m)
        if (lane + 32 * m < COLS) s_v[tt * COLS + lane + 32 * m] = v[q][m] * vmul;
    }
  };

  const int cg = (tid % DR_COMPUTE) / SPLIT, rs = tid % SPLIT;     // this lane's columns c0 + CB cg .., its rows rs + 8 n
  const int col = c0 + cg * CB;
  float* S = p.state + ((size_t)p.state_slots[seq] * p.H + h) * dk * dv;
  float s[RPT][CB];
  if (loader) {
    if (nchunks > 0) prepare(0);
  } else {
    const bool vec_state = CB == 4 && dv % 4 == 0 && ((uintptr_t)S & 15) == 0;
#pragma unroll
    for (int n = 0; n < RPT; ++n) {
      const int i = n * SPLIT + rs;
      if (vec_state) {
        const float4 x = (i < dk && col < dv) ? *reinterpret_cast<const float4*>(S + (size_t)i * dv + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        s[n][0] = x.x; s[n][CB > 1 ? 1 : 0] = x.y; s[n][CB > 2 ? 2 : 0] = x.z; s[n][CB > 3 ? 3 : 0] = x.w;
      } else {
#pragma unroll
        for (int c = 0; c < CB; ++c) s[n][c] = (i < dk && col + c < dv) ? S[(size_t)i * dv + col + c] : 0.f;
      }
    }
  }
  __syncthreads();
  for (int c = 0; c < nchunks; ++c) {
    if (loader) {
      if (c + 1 < nchunks) prepare(c + 1);
    } else {
      const float* b = sm + (c & 1) * buf_floats;
      const int t0 = t_begin + c * chunk, nt = min(chunk, t_end - t0);
#pragma unroll 2
      for (int tt = 0; tt < nt; ++tt) {
        const float* u = b + tt * DKP + rs;
        const float* d = u + chunk * DKP;
        const float* au = d + chunk * DKP;
        const float* k = au + chunk * DKP;
        const float* r = k + chunk * DKP;
        float vv[CB], us[CB], ut[CB], o[CB], o2[CB];
        if constexpr (CB == 4) {
          const float4 v = *reinterpret_cast<const float4*>(b + 5 * chunk * DKP + tt * COLS + cg * CB);
          vv[0] = v.x; vv[1] = v.y; vv[2] = v.z; vv[3] = v.w;
        } else {
#pragma unroll
          for (int cc = 0; cc < CB; ++cc) vv[cc] = b[5 * chunk * DKP + tt * COLS + cg * CB + cc];
        }
#pragma unroll
        for (int cc = 0; cc < CB; ++cc) us[cc] = ut[cc] = o[cc] = o2[cc] = 0.f;
        if (p.mode == 0) {
#pragma unroll
          for (int n = 0; n < RPT; n += 2) {
            const float ua = u[n * SPLIT], ub = u[(n + 1) * SPLIT];
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
              us[cc] = fmaf(ua, s[n][cc], us[cc]);
              ut[cc] = fmaf(ub, s[n + 1][cc], ut[cc]);
            }
          }
#pragma unroll
          for (int cc = 0; cc < CB; ++cc) {
            us[cc] += ut[cc];
#pragma unroll
            for (int w = 1; w < SPLIT; w <<= 1) us[cc] += __shfl_xor_sync(0xffffffffu, us[cc], w);
          }
#pragma unroll
          for (int n = 0; n < RPT; n += 2) {
            const float ka = k[n * SPLIT], kb = k[(n + 1) * SPLIT], aa = -au[n * SPLIT], ab = -au[(n + 1) * SPLIT];
            const float da = d[n * SPLIT], db = d[(n + 1) * SPLIT], ra = r[n * SPLIT], rb = r[(n + 1) * SPLIT];
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
              s[n][cc] = fmaf(ka, vv[cc], fmaf(aa, us[cc], da * s[n][cc]));
              s[n + 1][cc] = fmaf(kb, vv[cc], fmaf(ab, us[cc], db * s[n + 1][cc]));
              o[cc] = fmaf(s[n][cc], ra, o[cc]);
              o2[cc] = fmaf(s[n + 1][cc], rb, o2[cc]);
            }
          }
        } else if (p.mode == 1) {
          // one decay g and one rate for the whole head, and the key removed is the key written: the token's unit key
          // is read once and kept, S <- g S + k (beta v - beta g (k^T S))^T.  The loader left g and beta g in the first
          // two places of the row that holds u in the general form.
          const float g = b[tt * DKP], bg = b[tt * DKP + 1];
          float kr[RPT];
#pragma unroll
          for (int n = 0; n < RPT; n += 2) {
            kr[n] = k[n * SPLIT];
            kr[n + 1] = k[(n + 1) * SPLIT];
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
              us[cc] = fmaf(kr[n], s[n][cc], us[cc]);
              ut[cc] = fmaf(kr[n + 1], s[n + 1][cc], ut[cc]);
            }
          }
#pragma unroll
          for (int cc = 0; cc < CB; ++cc) {
            us[cc] += ut[cc];
#pragma unroll
            for (int w = 1; w < SPLIT; w <<= 1) us[cc] += __shfl_xor_sync(0xffffffffu, us[cc], w);
            us[cc] = fmaf(-bg, us[cc], vv[cc]);          // what is written along the key
          }
#pragma unroll
          for (int n = 0; n < RPT; n += 2) {
            const float ra = r[n * SPLIT], rb = r[(n + 1) * SPLIT];
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
              s[n][cc] = fmaf(kr[n], us[cc], g * s[n][cc]);
              s[n + 1][cc] = fmaf(kr[n + 1], us[cc], g * s[n + 1][cc]);
              o[cc] = fmaf(s[n][cc], ra, o[cc]);
              o2[cc] = fmaf(s[n + 1][cc], rb, o2[cc]);
            }
          }
        } else {
          // no removal: S <- diag(d) S + k v^T
#pragma unroll
          for (int n = 0; n < RPT; n += 2) {
            const float ka = k[n * SPLIT], kb = k[(n + 1) * SPLIT];
            const float da = d[n * SPLIT], db = d[(n + 1) * SPLIT], ra = r[n * SPLIT], rb = r[(n + 1) * SPLIT];
#pragma unroll
            for (int cc = 0; cc < CB; ++cc) {
              s[n][cc] = fmaf(ka, vv[cc], da * s[n][cc]);
              s[n + 1][cc] = fmaf(kb, vv[cc], db * s[n + 1][cc]);
              o[cc] = fmaf(s[n][cc], ra, o[cc]);
              o2[cc] = fmaf(s[n + 1][cc], rb, o2[cc]);
            }
          }
        }
        if constexpr (CB == 4) {
          // the four sums over eight lanes in four shuffles: halves of the values change hands, then quarters; lane rs
          // ends with the whole sum of column 2 (rs & 1) + ((rs >> 1) & 1)
          const bool odd = rs & 1, hi = rs & 2;
          float a0 = (odd ? o[2] + o2[2] : o[0] + o2[0]) + __shfl_xor_sync(0xffffffffu, odd ? o[0] + o2[0] : o[2] + o2[2], 1);
          float a1 = (odd ? o[3] + o2[3] : o[1] + o2[1]) + __shfl_xor_sync(0xffffffffu, odd ? o[1] + o2[1] : o[3] + o2[3], 1);
          float tot = (hi ? a1 : a0) + __shfl_xor_sync(0xffffffffu, hi ? a0 : a1, 2);
          tot += __shfl_xor_sync(0xffffffffu, tot, 4);
          const int mine = col + 2 * (rs & 1) + ((rs >> 1) & 1);
          if (rs < 4 && mine < dv) p.out[(size_t)(t0 + tt) * p.H * dv + h * dv + mine] = tot;
        } else {
#pragma unroll
          for (int cc = 0; cc < CB; ++cc) {
            float tot = o[cc] + o2[cc];
#pragma unroll
            for (int w = 1; w < SPLIT; w <<= 1) tot += __shfl_xor_sync(0xffffffffu, tot, w);
            if (rs == 0 && col + cc < dv) p.out[(size_t)(t0 + tt) * p.H * dv + h * dv + col + cc] = tot;
          }
        }
      }
    }
    __syncthreads();
  }
  pdl_launch_dependents();
  if (!loader) {
    const bool vec_state = CB == 4 && dv % 4 == 0 && ((uintptr_t)S & 15) == 0;
#pragma unroll
    for (int n = 0; n < RPT; ++n) {
      const int i = n * SPLIT + rs;
      if (vec_state) {
        if (i < dk && col < dv)
          *reinterpret_cast<float4*>(S + (size_t)i * dv + col) = make_float4(s[n][0], s[n][CB > 1 ? 1 : 0], s[n][CB > 2 ? 2 : 0], s[n][CB > 3 ? 3 : 0]);
      } else {
#pragma unroll
        for (int cc = 0; cc < CB; ++cc)
          if (i < dk && col + cc < dv) S[(size_t)i * dv + col + cc] = s[n][cc];
      }
    }
  }
}

// out[t, h*dv + j] = o[t, h, j] / sqrt(mean_j(o[t, h, :]^2) + eps) * gain[h*dv + j] * act(gate[t, h*dv + j]), act the sigmoid
// (gate_act 0) or z * sigmoid(z) (gate_act 1), or no gate at all (gate_act 2: `proj` is not read); a warp per (t, h).
template <typename TO>
__global__ void delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gain, const float* __restrict__ proj,
                                 int ld, int off_g, float eps, TO* __restrict__ out, int rows, int H, int dv, int gate_act,
                                 int out_ld, int out_off) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // (t, h)
  if (row >= rows) return;
  const int t = row / H, h = row % H;
  const float* x = o + (size_t)row * dv;
  float ss = 0.f;
  for (int j = lane; j < dv; j += 32) ss = fmaf(x[j], x[j], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* g = proj + (size_t)t * ld + off_g + h * dv;
  for (int j = lane; j < dv; j += 32) {
    const float gate = gate_act == 2 ? 1.0f : (gate_act == 1 ? g[j] * sigmoidf_(g[j]) : sigmoidf_(g[j]));
    out[(size_t)t * out_ld + out_off + h * dv + j] = from_f32<TO>(x[j] * inv * gain[h * dv + j] * gate);
  }
}

// the same with a CTA per (t, h): a "head" of many hundred channels (one norm over all of a row's heads together)
template <typename TO>
__global__ void __launch_bounds__(256)
delta_out_wide_kernel(const float* __restrict__ o, const float* __restrict__ gain, const float* __restrict__ proj, int ld, int off_g,
                      float eps, TO* __restrict__ out, int H, int dv, int gate_act, int out_ld, int out_off) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const int t = (int)(row / H), h = (int)(row % H);
  const float* x = o + row * dv;
  float ss = 0.f;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) ss = fmaf(x[j], x[j], ss);
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* g = proj + (size_t)t * ld + off_g + h * dv;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    const float gate = gate_act == 2 ? 1.0f : (gate_act == 1 ? g[j] * sigmoidf_(g[j]) : sigmoidf_(g[j]));
    out[(size_t)t * out_ld + out_off + h * dv + j] = from_f32<TO>(x[j] * inv * gain[h * dv + j] * gate);
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_delta_rule_supports(int dk, int dv) { return dk >= 1 && dk <= 256 && dv >= 1 && dv <= 65535 * 16; }

template <int RPT, int CB>
static int launch_delta_rule(DeltaParams p, int S, cudaStream_t stream) {
  constexpr int DKP = RPT * DR_SPLIT, DR_COLS = DR_COMPUTE / DR_SPLIT * CB;
  const size_t per_token = (size_t)(5 * DKP + DR_COLS) * sizeof(float);
  int chunk = (int)((96 * 1024) / (2 * per_token));
  chunk = chunk > DR_MAX_CHUNK ? DR_MAX_CHUNK : (chunk < 1 ? 1 : chunk);
  if (p.max_q > 0 && chunk > p.max_q) chunk = p.max_q;      // single decoded tokens: little shared memory, more CTAs an SM
  p.chunk = chunk;
  const size_t smem = 2 * per_token * chunk;
  static size_t allowed = 48 * 1024;          // (per instantiation: what the kernel has been told it may use)
  if (smem > allowed) {
    if (cudaFuncSetAttribute(delta_rule_kernel<RPT, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      set_error("delta_rule: the kernel's shared memory could not be raised");
      return SLLM_ERR_LAUNCH;
    }
    allowed = smem;
  }
  const dim3 grid((unsigned)S, (unsigned)p.H, (unsigned)((p.dv + DR_COLS - 1) / DR_COLS));
  launch_kernel(delta_rule_kernel<RPT, CB>, grid, DR_THREADS, smem, stream, p);
  return launch_status("delta_rule");
}

static int dispatch_delta_rule(DeltaParams p, int S, cudaStream_t stream);

SLLM_EXPORT int sllm_delta_rule(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* decay,
                                const float* a_bias, float* state, const int* q_start, const int* state_slots, float* out,
                                int S, int H, int dk, int dv, int max_q, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535, "delta_rule: bad sizes S=%d H=%d", S, H);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "delta_rule: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_r >= 0 && off_k >= 0 && off_v >= 0 && off_a >= 0 && off_r + H * dk <= ld && off_k + H * dk <= ld &&
                   off_v + H * dv <= ld && off_a + H * dk <= ld, "delta_rule: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = proj; p.decay = decay; p.a_bias = a_bias; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_r; p.off_k = off_k; p.off_v = off_v; p.off_a = off_a; p.H = H; p.dk = dk; p.dv = dv;
  p.chunk = 1;
  p.max_q = max_q;           // the longest portion of the batch (0: not known)
  p.mode = 0; p.hdiv = 1; p.gates = nullptr; p.ldg = p.off_b = p.off_dt = 0; p.a_log = p.dt_bias = nullptr;
  p.r_scale = 1.f; p.inv_tau = 1.f;
  return dispatch_delta_rule(p, S, stream);
}

static int dispatch_delta_rule(DeltaParams p, int S, cudaStream_t stream) {
  const int dk = p.dk, dv = p.dv;
  // enough (request, head, 64 columns) for every SM: four columns a lane; else one, in four times the CTAs
  const bool wide = (long)S * p.H * ((dv + 63) / 64) >= (long)num_sms();
#define SLLM_DR(RPT_) return wide ? launch_delta_rule<RPT_, 4>(p, S, stream) : launch_delta_rule<RPT_, 1>(p, S, stream)
  if (dk <= 16) SLLM_DR(2);
  if (dk <= 32) SLLM_DR(4);
  if (dk <= 64) SLLM_DR(8);
  if (dk <= 128) SLLM_DR(16);
  SLLM_DR(32);
#undef SLLM_DR
}

// The gated delta rule over conv'd, activated q | k | v columns of `qkv` [T, ld] (query/key heads Hk, value heads H) with
// one beta logit and one decay logit per head in `gates` [T, ldg].
SLLM_EXPORT int sllm_gated_delta_rule(const float* qkv, int ld, int off_q, int off_k, int off_v, const float* gates, int ldg,
                                      int off_b, int off_dt, const float* a_log, const float* dt_bias, float* state,
                                      const int* q_start, const int* state_slots, float* out, int S, int H, int Hk, int dk, int dv,
                                      float q_scale, int max_q, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535 && Hk > 0 && H % Hk == 0, "gated_delta_rule: bad sizes S=%d H=%d Hk=%d", S, H, Hk);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "gated_delta_rule: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_q >= 0 && off_k >= 0 && off_v >= 0 && off_q + Hk * dk <= ld && off_k + Hk * dk <= ld && off_v + H * dv <= ld,
               "gated_delta_rule: columns outside the product's %d", ld);
  SLLM_REQUIRE(off_b >= 0 && off_dt >= 0 && off_b + H <= ldg && off_dt + H <= ldg, "gated_delta_rule: gate columns outside %d", ldg);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = qkv; p.decay = qkv; p.a_bias = nullptr; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_q; p.off_k = off_k; p.off_v = off_v; p.off_a = 0; p.H = H; p.dk = dk; p.dv = dv;
  p.chunk = 1; p.max_q = max_q;
  p.mode = 1; p.hdiv = H / Hk; p.gates = gates; p.ldg = ldg; p.off_b = off_b; p.off_dt = off_dt; p.a_log = a_log; p.dt_bias = dt_bias;
  p.r_scale = q_scale; p.inv_tau = 1.f;
  return dispatch_delta_rule(p, S, stream);
}

// Gated linear attention over q | k | v columns of `proj` [T, ld] with decay logits `z` [T, H*dk]: alpha = sigmoid(z)^(inv_tau).
SLLM_EXPORT int sllm_gated_linear_attention(const float* proj, int ld, int off_q, int off_k, int off_v, const float* z,
                                            float* state, const int* q_start, const int* state_slots, float* out, int S, int H,
                                            int dk, int dv, float q_scale, float inv_tau, int max_q, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535, "gated_linear_attention: bad sizes S=%d H=%d", S, H);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "gated_linear_attention: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_q >= 0 && off_k >= 0 && off_v >= 0 && off_q + H * dk <= ld && off_k + H * dk <= ld && off_v + H * dv <= ld,
               "gated_linear_attention: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = proj; p.decay = z; p.a_bias = nullptr; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_q; p.off_k = off_k; p.off_v = off_v; p.off_a = 0; p.H = H; p.dk = dk; p.dv = dv;
  p.chunk = 1; p.max_q = max_q;
  p.mode = 2; p.hdiv = 1; p.gates = nullptr; p.ldg = p.off_b = p.off_dt = 0; p.a_log = p.dt_bias = nullptr;
  p.r_scale = q_scale; p.inv_tau = inv_tau;
  return dispatch_delta_rule(p, S, stream);
}

// Linear attention with a fixed decay per head (`decay` [H]) over silu'd q | k | v columns of `proj` [T, ld].
SLLM_EXPORT int sllm_decay_linear_attention(const float* proj, int ld, int off_q, int off_k, int off_v, const float* decay,
                                            float* state, const int* q_start, const int* state_slots, float* out, int S, int H,
                                            int dk, int dv, int max_q, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535, "decay_linear_attention: bad sizes S=%d H=%d", S, H);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "decay_linear_attention: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_q >= 0 && off_k >= 0 && off_v >= 0 && off_q + H * dk <= ld && off_k + H * dk <= ld && off_v + H * dv <= ld,
               "decay_linear_attention: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = proj; p.decay = proj; p.a_bias = nullptr; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_q; p.off_k = off_k; p.off_v = off_v; p.off_a = 0; p.H = H; p.dk = dk; p.dv = dv;
  p.chunk = 1; p.max_q = max_q;
  p.mode = 3; p.hdiv = 1; p.gates = nullptr; p.ldg = p.off_b = p.off_dt = 0; p.a_log = decay; p.dt_bias = nullptr;
  p.r_scale = 1.f; p.inv_tau = 1.f;
  return dispatch_delta_rule(p, S, stream);
}

// Linear attention whose forget gate also writes, over q | gate logit | v columns of `proj` [T, ld]: `f_bias` and `lower` [H*dk].
SLLM_EXPORT int sllm_forget_gate_attention(const float* proj, int ld, int off_q, int off_f, int off_v, const float* f_bias,
                                           const float* lower, float* state, const int* q_start, const int* state_slots,
                                           float* out, int S, int H, int dk, int dv, int max_q, cudaStream_t stream) {
  SLLM_REQUIRE(S >= 0 && H > 0 && H <= 65535, "forget_gate_attention: bad sizes S=%d H=%d", S, H);
  SLLM_REQUIRE(sllm_delta_rule_supports(dk, dv), "forget_gate_attention: a head of %d key and %d value channels is outside 1..256 keys", dk, dv);
  SLLM_REQUIRE(off_q >= 0 && off_f >= 0 && off_v >= 0 && off_q + H * dk <= ld && off_f + H * dk <= ld && off_v + H * dv <= ld,
               "forget_gate_attention: columns outside the product's %d", ld);
  if (S == 0) return SLLM_OK;
  DeltaParams p;
  p.proj = proj; p.decay = proj; p.a_bias = f_bias; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.out = out; p.ld = ld; p.off_r = off_q; p.off_k = off_f; p.off_v = off_v; p.off_a = 0; p.H = H; p.dk = dk; p.dv = dv;
  p.chunk = 1; p.max_q = max_q;
  p.mode = 4; p.hdiv = 1; p.gates = nullptr; p.ldg = p.off_b = p.off_dt = 0; p.a_log = lower; p.dt_bias = nullptr;
  p.r_scale = 1.f; p.inv_tau = 1.f;
  return dispatch_delta_rule(p, S, stream);
}

SLLM_EXPORT int sllm_delta_out(const float* o, const float* gain, const float* proj, int ld, int off_g, float eps, void* out,
                               int out_dtype, int T, int H, int dv, int gate_act, int out_ld, int out_off, cudaStream_t stream) {
  SLLM_REQUIRE(out_off >= 0 && out_off + H * dv <= out_ld, "delta_out: the output's columns lie outside its %d", out_ld);
  SLLM_REQUIRE(T >= 0 && H > 0 && dv > 0 && (gate_act == 2 || (off_g >= 0 && off_g + H * dv <= ld)), "delta_out: bad sizes T=%d H=%d dv=%d", T, H, dv);
  if (T == 0) return SLLM_OK;
  const long rows = (long)T * H;
  if (dv >= 512) {                      // a warp would walk such a row sixteen times and more
    if (out_dtype == SLLM_F32)
      launch_kernel(delta_out_wide_kernel<float>, (unsigned)rows, 256, 0, stream, o, gain, proj, ld, off_g, eps, (float*)out, H, dv, gate_act, out_ld, out_off);
    else if (out_dtype == SLLM_BF16)
      launch_kernel(delta_out_wide_kernel<__nv_bfloat16>, (unsigned)rows, 256, 0, stream, o, gain, proj, ld, off_g, eps,
                    (__nv_bfloat16*)out, H, dv, gate_act, out_ld, out_off);
    else
      SLLM_REQUIRE(false, "delta_out: unknown dtype %d", out_dtype);
    return launch_status("delta_out");
  }
  const int blocks = (int)((rows + 7) / 8);
  if (out_dtype == SLLM_F32)
    launch_kernel(delta_out_kernel<float>, blocks, 256, 0, stream, o, gain, proj, ld, off_g, eps, (float*)out, (int)rows, H, dv, gate_act, out_ld, out_off);
  else if (out_dtype == SLLM_BF16)
    launch_kernel(delta_out_kernel<__nv_bfloat16>, blocks, 256, 0, stream, o, gain, proj, ld, off_g, eps, (__nv_bfloat16*)out,
                  (int)rows, H, dv, gate_act, out_ld, out_off);
  else
    SLLM_REQUIRE(false, "delta_out: unknown dtype %d", out_dtype);
  return launch_status("delta_out");
}
