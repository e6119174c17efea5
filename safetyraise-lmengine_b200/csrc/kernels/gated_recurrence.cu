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
//                       Long portions of the bfloat16 engine: in 32 segments side by side (see below).
#include "common.cuh"

namespace srlm {

constexpr int GN = 64, GK = 16;      // outputs and k of a tile of the gates' products; TT tokens a tile, TT / 16 a thread

template <typename TW, int TT>
__global__ void __launch_bounds__(256)
recurrence_gates_kernel(const float* __restrict__ u, const TW* __restrict__ Ra, const TW* __restrict__ Ri,
                        const float* __restrict__ ba, const float* __restrict__ bi, const float* __restrict__ rate,
                        float* __restrict__ a_out, float* __restrict__ b_out, int T, int C, int Cb) {
  pdl_wait();
  pdl_trigger();
  constexpr int PT = TT / 16;                               // tokens a thread
  constexpr int UL = TT * GK / 256 > 0 ? TT * GK / 256 : 1; // elements of the token tile a thread fetches
  __shared__ __align__(16) float Us[GK][TT + 4];
  __shared__ __align__(16) float Wa[GK][GN + 4];
  __shared__ __align__(16) float Wi[GK][GN + 4];
  const int blk = blockIdx.y, n0 = blockIdx.x * GN, t0 = blockIdx.z * TT;
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;                   // PT tokens x 4 outputs a thread
  const TW* Rab = Ra + (size_t)blk * Cb * Cb;
  const TW* Rib = Ri + (size_t)blk * Cb * Cb;
  float acc_a[PT][4] = {}, acc_i[PT][4] = {};
  // a thread's share of a k-slab, fetched into registers one slab ahead of the arithmetic
  float ur[UL], war[4], wir[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int x = 0; x < UL; ++x) {
      const int idx = tid + x * 256;
      const int r = idx / GK, c = idx % GK;
      const int t = t0 + r, k = k0 + c;
      ur[x] = (idx < TT * GK && t < T && k < Cb) ? u[(size_t)t * C + (size_t)blk * Cb + k] : 0.f;
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int idx = tid + x * 256;
      const int r = idx / GK, c = idx % GK;
      const int n = n0 + r, k = k0 + c;
      const bool ok = n < Cb && k < Cb;
      war[x] = ok ? to_float(Rab[(size_t)n * Cb + k]) : 0.f;
      wir[x] = ok ? to_float(Rib[(size_t)n * Cb + k]) : 0.f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < Cb; k0 += GK) {
#pragma unroll
    for (int x = 0; x < UL; ++x) {
      const int idx = tid + x * 256;
      if (idx < TT * GK) Us[idx % GK][idx / GK] = ur[x];
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int idx = tid + x * 256;
      Wa[idx % GK][idx / GK] = war[x];
      Wi[idx % GK][idx / GK] = wir[x];
    }
    __syncthreads();
    if (k0 + GK < Cb) fetch(k0 + GK);
#pragma unroll
    for (int kk = 0; kk < GK; ++kk) {
      float uv[PT];
      if constexpr (PT % 4 == 0) {
#pragma unroll
        for (int i = 0; i < PT; i += 4) {
          const float4 u4 = *reinterpret_cast<const float4*>(&Us[kk][ty * PT + i]);
          uv[i] = u4.x; uv[i + 1] = u4.y; uv[i + 2] = u4.z; uv[i + 3] = u4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < PT; ++i) uv[i] = Us[kk][ty * PT + i];
      }
      const float4 wa = *reinterpret_cast<const float4*>(&Wa[kk][tx * 4]);
      const float4 wi = *reinterpret_cast<const float4*>(&Wi[kk][tx * 4]);
#pragma unroll
      for (int i = 0; i < PT; ++i) {
        acc_a[i][0] = fmaf(uv[i], wa.x, acc_a[i][0]);
        acc_a[i][1] = fmaf(uv[i], wa.y, acc_a[i][1]);
        acc_a[i][2] = fmaf(uv[i], wa.z, acc_a[i][2]);
        acc_a[i][3] = fmaf(uv[i], wa.w, acc_a[i][3]);
        acc_i[i][0] = fmaf(uv[i], wi.x, acc_i[i][0]);
        acc_i[i][1] = fmaf(uv[i], wi.y, acc_i[i][1]);
        acc_i[i][2] = fmaf(uv[i], wi.z, acc_i[i][2]);
        acc_i[i][3] = fmaf(uv[i], wi.w, acc_i[i][3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < PT; ++i) {
    const int t = t0 + ty * PT + i;
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

constexpr int kAhead = 8;     // tokens whose operands a thread requests before it walks them

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

// The same walk for long portions, in segments: thread (channel, segment) walks its share of an entry's tokens from zero
// and keeps the product of its decays; the segments' starts follow from these by a short fold over the segments before;
// then every thread walks its share again from its true start and writes.  The sums are formed in another order than
// token by token (rounding only), so the engine's float32 path, whose logits do not depend on the cutting, keeps to the
// walk above.
constexpr int kSegs = 32;

template <typename TO>
__global__ void __launch_bounds__(32 * kSegs)
linear_recurrence_segments_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ y,
                                  long long ldy, const float* __restrict__ y_bias, float* __restrict__ state,
                                  long long state_stride, const int* __restrict__ cu_q, const int* __restrict__ slots,
                                  TO* __restrict__ out, int C) {
  pdl_wait();
  pdl_trigger();
  __shared__ float As[kSegs][33], Bs[kSegs][33];
  const int e = blockIdx.y, seg = threadIdx.y;
  const int c = blockIdx.x * 32 + threadIdx.x;
  const bool live = c < C;
  const int first = cu_q[e], n = cu_q[e + 1] - first;
  const int L = (n + kSegs - 1) / kSegs;
  const int lo = min(n, seg * L), hi = min(n, lo + L);
  float A = 1.f, B = 0.f;
  if (live) {
    for (int t0 = lo; t0 < hi; t0 += 8) {
      float av[8], bv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool ok = t0 + j < hi;
        const size_t t = (size_t)(first + (ok ? t0 + j : lo));
        av[j] = ok ? a[t * C + c] : 1.f;
        bv[j] = ok ? b[t * C + c] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        B = fmaf(av[j], B, bv[j]);
        A *= av[j];
      }
    }
  }
  As[seg][threadIdx.x] = A;
  Bs[seg][threadIdx.x] = B;
  __syncthreads();
  if (!live) return;
  float* s_g = state + (size_t)slots[e] * state_stride + c;
  float S = *s_g;
  for (int sg = 0; sg < seg; ++sg) S = fmaf(As[sg][threadIdx.x], S, Bs[sg][threadIdx.x]);
  const float yb = y_bias ? y_bias[c] : 0.f;
  for (int t0 = lo; t0 < hi; t0 += 8) {
    float av[8], bv[8], yv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool ok = t0 + j < hi;
      const size_t t = (size_t)(first + (ok ? t0 + j : lo));
      av[j] = ok ? a[t * C + c] : 1.f;
      bv[j] = ok ? b[t * C + c] : 0.f;
      yv[j] = ok ? y[t * ldy + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (t0 + j >= hi) break;
      S = fmaf(av[j], S, bv[j]);
      out[(size_t)(first + t0 + j) * C + c] = from_float<TO>(S * gelu_tanh_g(yv[j] + yb));
    }
  }
  if (seg == kSegs - 1) *s_g = S;          // the last segment ends at the entry's last token (or is empty: the fold of all)
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
  const int tt = T > 16 ? 64 : 16;           // token tile: steps of a few tokens run one token a thread (tiles of 128
                                             // tokens, eight a thread, measured slower: 183 registers, one block an SM)
  dim3 grid((unsigned)((Cb + GN - 1) / GN), (unsigned)blocks, (unsigned)((T + tt - 1) / tt));
  if (grid.z > 65535) return refuse(ST_BAD_SIZE, "recurrence_gates: %d tokens", T);
  if (tt == 64)
    SRLM_DISPATCH_ACT(w_dtype, TW, launch_pdl(recurrence_gates_kernel<TW, 64>, grid, dim3(256), 0, stream, u, (const TW*)Ra,
                                              (const TW*)Ri, ba, bi, rate, a_out, b_out, T, C, Cb));
  else
    SRLM_DISPATCH_ACT(w_dtype, TW, launch_pdl(recurrence_gates_kernel<TW, 16>, grid, dim3(256), 0, stream, u, (const TW*)Ra,
                                              (const TW*)Ri, ba, bi, rate, a_out, b_out, T, C, Cb));
  return launched();
}

// a, b float32 [T, C]; y float32 [T, ldy] (the gate branch's columns from y), y_bias float32 [C] or null;
// state float32 [slots, state_stride] with S in its first C places; out [T, C].  in_segments: long portions, every
// entry's tokens cut into 32 segments that are walked side by side (another order of the sums: not for the float32 path)
extern "C" int srlm_linear_recurrence(const float* a, const float* b, const float* y, long long ldy, const float* y_bias,
                                      float* state, long long state_stride, const int* cu_q, const int* slots, void* out,
                                      int out_dtype, int n_entries, int C, int in_segments, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (C <= 0 || ldy < C || state_stride < C || n_entries > 65535)
    return refuse(ST_BAD_SIZE, "linear_recurrence: channels=%d ld=%lld", C, ldy);
  if (in_segments) {
    dim3 grid((unsigned)((C + 31) / 32), (unsigned)n_entries);
    SRLM_DISPATCH_ACT(out_dtype, TO, launch_pdl(linear_recurrence_segments_kernel<TO>, grid, dim3(32, kSegs), 0, stream, a, b,
                                                y, ldy, y_bias, state, state_stride, cu_q, slots, (TO*)out, C));
    return launched();
  }
  const int threads = 64;
  dim3 grid((unsigned)((C + threads - 1) / threads), (unsigned)n_entries);
  SRLM_DISPATCH_ACT(out_dtype, TO, launch_pdl(linear_recurrence_kernel<TO>, grid, dim3(threads), 0, stream, a, b, y, ldy,
                                              y_bias, state, state_stride, cu_q, slots, (TO*)out, C));
  return launched();
}
