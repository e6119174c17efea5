// A gated linear recurrence per channel:
//
//   r = logistic(R_a u + b_a);   i = logistic(R_i u + b_i)          R block-diagonal: B square blocks of C / B channels
//   a = exp(-rate r);   S <- a S + sqrt(1 - a^2) i u;   out = S * gelu_tanh(y + b_y)
//
// with rate[c] = decay_scale * softplus(lam[c]) formed once on the host side, u the convolved branch (float32 [T, C]) and y
// the gate branch's projection.  Everything is float32; 1 - a^2 is formed as -expm1(2 log a), which keeps its digits
// when a is close to one.
//
//   recurrence_gates    the two block-diagonal products (FMA, k in index order: a token's sums do not depend on its
//                       tile or on the batch) with the logistics, a and the scaled input in the epilogue:
//                       a [T, C] and b = sqrt(1 - a^2) i u [T, C]
//   linear_recurrence   S <- a S + b token by token, a thread a channel, the loads of several tokens in flight; the
//                       gate branch in the same pass; the slot's S renewed at the end.  S [C] leads the slot's row.
#include "common.cuh"

namespace srlm {

constexpr int GT = 32, GN = 64, GK = 16;      // tokens, outputs and k of a tile of the gates' products

template <typename TW>
__global__ void __launch_bounds__(256)
recurrence_gates_kernel(const float* __restrict__ u, const TW* __restrict__ Ra, const TW* __restrict__ Ri,
                        const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ rate,
                        float* __restrict__ a_out, float* __restrict__ b_out, int T, int C, int Cb) {
  pdl_wait();
  pdl_trigger();
  __shared__ float Us[GK][GT + 1];
  __shared__ float Wa[GK][GN + 1];
  __shared__ float Wi[GK][GN + 1];
  const int blk = blockIdx.y, n0 = blockIdx.x * GN, t0 = blockIdx.z * GT;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;                   // 2 tokens x 4 outputs a thread
  const TW* Rab = Ra + (size_t)blk * Cb * Cb;
  const TW* Rib = Ri + (size_t)blk * Cb * Cb;
  float acc_a[2][4] = {}, acc_i[2][4] = {};
  for (int k0 = 0; k0 < Cb; k0 += GK) {
    for (int idx = tid; idx < GT * GK; idx += 256) {
      const int r = idx / GK, c = idx % GK;
      const int t = t0 + r, k = k0 + c;
      Us[c][r] = (t < T && k < Cb) ? u[(size_t)t * C + (size_t)blk * Cb + k] : 0.f;
    }
    for (int idx = tid; idx < GN * GK; idx += 256) {
      const int r = idx / GK, c = idx % GK;
      const int n = n0 + r, k = k0 + c;
      const bool ok = n < Cb && k < Cb;
      Wa[c][r] = ok ? to_float(Rab[(size_t)n * Cb + k]) : 0.f;
      Wi[c][r] = ok ? to_float(Rib[(size_t)n * Cb + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      const float u0 = Us[kk][ty * 2], u1 = Us[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float wa = Wa[kk][tx * 4 + j], wi = Wi[kk][tx * 4 + j];
        acc_a[0][j] = fmaf(u0, wa, acc_a[0][j]);
        acc_a[1][j] = fmaf(u1, wa, acc_a[1][j]);
        acc_i[0][j] = fmaf(u0, wi, acc_i[0][j]);
        acc_i[1][j] = fmaf(u1, wi, acc_i[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int t = t0 + ty * 2 + i;
    if (t >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= Cb) continue;
      const int c = blk * Cb + n;
      const float r = 1.f / (1.f + expf(-(acc_a[i][j] + ba[c])));
      const float g = 1.f / (1.f + expf(-(acc_i[i][j] + bi[c])));
      const float log_a = -rate[c] * r;
      a_out[(size_t)t * C + c] = expf(log_a);
      b_out[(size_t)t * C + c] = sqrtf(-expm1f(2.f * log_a)) * g * u[(size_t)t * C + c];
    }
  }
}

__device__ __forceinline__ float gelu_tanh_g(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

constexpr int kAhead = 4;     // tokens whose operands a thread requests before it walks them

template <typename TO>
__global__ void linear_recurrence_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                         const float* __restrict__ y, long long ldy, const float* __restrict__ y_bias,
                                         float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                                         const int* __restrict__ slots, TO* __restrict__ out, int C) {
  pdl_wait();
  pdl_trigger();
  const int e = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int first = cu_q[e], n = cu_q[e + 1] - first;
  float* s_g = state + (size_t)slots[e] * state_stride + c;
  float S = *s_g;
  const float yb = y_bias ? y_bias[c] : 0.f;
  for (int t0 = 0; t0 < n; t0 += kAhead) {
    float av[kAhead], bv[kAhead], yv[kAhead];
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const bool ok = t0 + j < n;
      const size_t t = (size_t)(first + t0 + (ok ? j : 0));
      av[j] = ok ? a[t * C + c] : 1.f;
      bv[j] = ok ? b[t * C + c] : 0.f;
      yv[j] = ok ? y[t * ldy + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      if (t0 + j >= n) break;
      S = fmaf(av[j], S, bv[j]);
      out[(size_t)(first + t0 + j) * C + c] = from_float<TO>(S * gelu_tanh_g(yv[j] + yb));
    }
  }
  *s_g = S;
}

}  // namespace srlm

using namespace srlm;

// u float32 [T, C]; Ra, Ri [B, C / B, C / B] ([out, in], w_dtype); ba, bi, rate float32 [C]; a_out, b_out float32 [T, C]
extern "C" int srlm_recurrence_gates(const float* u, const void* Ra, const void* Ri, int w_dtype, const float* ba,
                                     const float* bi, const float* rate, float* a_out, float* b_out, int T, int C,
                                     int blocks, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (C <= 0 || blocks <= 0 || C % blocks || blocks > 65535)
    return refuse(ST_BAD_SIZE, "recurrence_gates: %d channels in %d blocks", C, blocks);
  const int Cb = C / blocks;
  dim3 grid((unsigned)((Cb + GN - 1) / GN), (unsigned)blocks, (unsigned)((T + GT - 1) / GT));
  if (grid.z > 65535) return refuse(ST_BAD_SIZE, "recurrence_gates: %d tokens", T);
  SRLM_DISPATCH_ACT(w_dtype, TW, launch_pdl(recurrence_gates_kernel<TW>, grid, dim3(256), 0, stream, u, (const TW*)Ra,
                                            (const TW*)Ri, ba, bi, rate, a_out, b_out, T, C, Cb));
  return launched();
}

// a, b float32 [T, C]; y float32 [T, ldy] (the gate branch's columns from y), y_bias float32 [C] or null;
// state float32 [slots, state_stride] with S in its first C places; out [T, C]
extern "C" int srlm_linear_recurrence(const float* a, const float* b, const float* y, long long ldy, const float* y_bias,
                                      float* state, long long state_stride, const int* cu_q, const int* slots, void* out,
                                      int out_dtype, int n_entries, int C, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (C <= 0 || ldy < C || state_stride < C || n_entries > 65535)
    return refuse(ST_BAD_SIZE, "linear_recurrence: channels=%d ld=%lld", C, ldy);
  const int threads = 64;
  dim3 grid((unsigned)((C + threads - 1) / threads), (unsigned)n_entries);
  SRLM_DISPATCH_ACT(out_dtype, TO, launch_pdl(linear_recurrence_kernel<TO>, grid, dim3(threads), 0, stream, a, b, y, ldy,
                                              y_bias, state, state_stride, cu_q, slots, (TO*)out, C));
  return launched();
}
