// The selective scan: a recurrent mixer with a state S [channels, N] per request, written and read token by token.
//
//   x <- silu(conv(x) + conv_bias)         a short causal convolution per channel over time (zeros before the start)
//   dt = softplus(dt_raw + dt_bias)        per channel; dt_raw is a projection of the token
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n
//   y_c = sum_n S[c, n] C_n + D_c x_c;     out_c = y_c * silu(z_c)
//
// A (negative), D per channel and the biases are float32; B and C [N] come per token from a projection of x.  What a
// request carries from step to step lies in its slot, float32: S of every channel, then the last taps - 1 inputs of
// every channel's convolution.  Everything here is float32 arithmetic; only `out` (the input of the output product)
// and the optional second copy of x (the input of the B / C / dt product) are written in the activation dtype.
//
//   conv   one thread per (token, four neighbouring channels; one where rows do not allow 16-byte accesses): reads
//          the step's inputs, and the slot's carried inputs for the first taps - 1 tokens of an entry
//   scan   one block per (entry, 16 channels): four warps walk the entry's tokens in order, 8 lanes sharing a channel's
//          N states, through chunks of 16 tokens in shared memory; the lanes' partial sums of 8 tokens are added in
//          one exchange of 7 shuffles.  Four more warps fetch the chunks several ahead (cp.async), form the step
//          sizes, and gate and write a finished chunk's y as a block; at the end the walkers renew the slot's S and
//          carried inputs.
//          A channel's sums do not depend on what else is in the step or on how the tokens were cut into steps.
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace srlm {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// state of a slot: [channels * N] S, then [channels * (taps - 1)] carried inputs, oldest first
template <typename TL, int V>
__global__ void scan_conv_kernel(const float* __restrict__ xz, long long ld, const float* __restrict__ conv_w,
                                 const float* __restrict__ conv_b, const float* __restrict__ state, long long state_stride,
                                 const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                                 const int* __restrict__ slots, float* __restrict__ x_out, TL* __restrict__ x_low,
                                 int T, int channels, int N, int taps) {
  pdl_wait();
  pdl_trigger();
  const int per_token = channels / V;                      // V neighbouring channels a thread (V divides channels)
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * per_token) return;
  const int t = (int)(idx / per_token), c = (int)(idx - (long long)t * per_token) * V;
  const int e = entry_of_token[t];
  const int i = t - cu_q[e];                               // the token's place in its entry
  const float* carry = state + (size_t)slots[e] * state_stride + (size_t)channels * N + (size_t)c * (taps - 1);
  float acc[V], v[V];
#pragma unroll
  for (int u = 0; u < V; ++u) acc[u] = conv_b ? conv_b[c + u] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;                         // tap j weighs the input `back` tokens ago
    if (back <= i) {
      const float* src = xz + (size_t)(t - back) * ld + c;
      if constexpr (V == 4) {
        const float4 f = *reinterpret_cast<const float4*>(src);
        v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
      } else {
#pragma unroll
        for (int u = 0; u < V; ++u) v[u] = src[u];
      }
    } else {
#pragma unroll
      for (int u = 0; u < V; ++u) v[u] = carry[(size_t)u * (taps - 1) + taps - 1 + i - back];
    }
#pragma unroll
    for (int u = 0; u < V; ++u) acc[u] = fmaf(conv_w[(size_t)(c + u) * taps + j], v[u], acc[u]);
  }
#pragma unroll
  for (int u = 0; u < V; ++u) acc[u] = silu_f(acc[u]);
  const size_t at = (size_t)t * channels + c;
  if constexpr (V == 4) {
    *reinterpret_cast<float4*>(x_out + at) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  } else {
#pragma unroll
    for (int u = 0; u < V; ++u) x_out[at + u] = acc[u];
  }
  if (x_low) {
    if constexpr (V == 4 && sizeof(TL) == 2) {               // four 16-bit values in one 8-byte store
      TL low[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) low[u] = from_float<TL>(acc[u]);
      *reinterpret_cast<uint2*>(x_low + at) = *reinterpret_cast<const uint2*>(low);
    } else {
#pragma unroll
      for (int u = 0; u < V; ++u) x_low[at + u] = from_float<TL>(acc[u]);
    }
  }
}

// The same convolution for rows that allow 16-byte accesses and 2 to 4 taps: a thread owns four neighbouring channels
// over a run of tokens, holds their weights and the rows of the last TAPS - 1 tokens in registers, and reads every
// row once.  The sums are formed in the order of the kernel above (bias, then the taps from the oldest on).
template <typename TL, int TAPS>
__global__ void scan_conv_rows_kernel(const float* __restrict__ xz, long long ld, const float* __restrict__ conv_w,
                                      const float* __restrict__ conv_b, const float* __restrict__ state,
                                      long long state_stride, const int* __restrict__ entry_of_token,
                                      const int* __restrict__ cu_q, const int* __restrict__ slots,
                                      float* __restrict__ x_out, TL* __restrict__ x_low, int T, int channels, int N,
                                      int run) {
  pdl_wait();
  pdl_trigger();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= channels) return;
  const int t_begin = blockIdx.y * run, t_end = min(T, t_begin + run);
  float w[4][TAPS], bias[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    bias[u] = conv_b ? conv_b[c + u] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[u][j] = conv_w[(size_t)(c + u) * TAPS + j];
  }
  float4 prev[TAPS - 1];                                   // prev[k]: the row of token t - (TAPS - 1) + k
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) {
    const int row = t_begin - (TAPS - 1) + k;
    prev[k] = row >= 0 ? *reinterpret_cast<const float4*>(xz + (size_t)row * ld + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll 4
  for (int t = t_begin; t < t_end; ++t) {
    const int e = entry_of_token[t];
    const int i = t - cu_q[e];                             // the token's place in its entry
    const float4 cur = *reinterpret_cast<const float4*>(xz + (size_t)t * ld + c);
    float acc[4] = {bias[0], bias[1], bias[2], bias[3]};
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int back = TAPS - 1 - j;                       // tap j weighs the input `back` tokens ago
      float v[4];
      if (back <= i) {                                     // a row of this step (and of this entry)
        const float4 f = back == 0 ? cur : prev[j];
        v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
      } else {                                             // ahead of the portion: the slot's carried inputs
        const float* carry = state + (size_t)slots[e] * state_stride + (size_t)channels * N + (size_t)c * (TAPS - 1);
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = carry[(size_t)u * (TAPS - 1) + TAPS - 1 + i - back];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = fmaf(w[u][j], v[u], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = silu_f(acc[u]);
    const size_t at = (size_t)t * channels + c;
    *reinterpret_cast<float4*>(x_out + at) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    if (x_low) {
      if constexpr (sizeof(TL) == 2) {
        TL low[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) low[u] = from_float<TL>(acc[u]);
        *reinterpret_cast<uint2*>(x_low + at) = *reinterpret_cast<const uint2*>(low);
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) x_low[at + u] = from_float<TL>(acc[u]);
      }
    }
#pragma unroll
    for (int k = 0; k + 1 < TAPS - 1; ++k) prev[k] = prev[k + 1];
    prev[TAPS - 2] = cur;
  }
}

constexpr int kScanLanes = 8, kScanChannels = 16, kScanChunk = 16;

__device__ __forceinline__ void scan_cp_async_4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void scan_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void scan_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr float kLog2e = 1.4426950408889634f;

// 2^x for x <= 0 (a decay): the hardware's approximation, 2 ulp, zero below 2^-126
__device__ __forceinline__ float scan_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// n neighbouring floats of shared memory (n a power of two; the address a multiple of min(n, 4) floats)
template <int NPL>
__device__ __forceinline__ void scan_load_row(const float* src, float (&dst)[NPL]) {
  if constexpr (NPL == 1) {
    dst[0] = src[0];
  } else if constexpr (NPL == 2) {
    const float2 f = *reinterpret_cast<const float2*>(src);
    dst[0] = f.x, dst[1] = f.y;
  } else {
#pragma unroll
    for (int k = 0; k < NPL; k += 4) {
      const float4 f = *reinterpret_cast<const float4*>(src + k);
      dst[k] = f.x, dst[k + 1] = f.y, dst[k + 2] = f.z, dst[k + 3] = f.w;
    }
  }
}

// A chunk of 16 tokens lies in shared memory while the block walks it: B and C of every token, zero behind N up to
// the lanes' reach; per (token, channel) dt (raw, then its softplus), x, z; and the block's y ahead of the gate.
// Places behind an entry's last token hold dt = 0, x = 0, B = 0: S <- fma(1, S, 0) leaves every state as it is, so
// the walk has no branch.
//
// The block's first four warps walk; its other four fetch, prepare and finish.  While the walkers are on chunk j the
// helpers wait for chunk j + 1 (cp.async), turn its raw step sizes into softplus(dt + bias), gate and write the y of
// chunk j - 1, and issue the fetch of chunk j + K - 1 into the buffer chunk j - 1 has left: K buffers of operands
// (a fetch has K - 2 walks of a chunk to arrive: a chunk's walk is shorter than a trip to DRAM), two of y, one
// barrier a chunk.  Every round commits one group of copies, an empty one behind the entry's end, so that "all but
// the last K - 3 groups" always names chunk j + 1.  A helper prepares and finishes exactly the (token, channel)
// places it fetched, so only the barrier orders helpers and walkers.
constexpr int kScanWalkers = kScanLanes * kScanChannels, kScanThreads = 2 * kScanWalkers;
constexpr int scan_buffers(int npl) { return npl <= 2 ? 6 : npl <= 4 ? 5 : 4; }

template <typename TO, int NPL>
__global__ void __launch_bounds__(kScanThreads)
selective_scan_kernel(const float* __restrict__ x, const float* __restrict__ xz, long long ld_xz,
                      const float* __restrict__ dbc, long long ld_dbc, int b_off, const float* __restrict__ dt_raw,
                      const float* __restrict__ dt_bias, const float* __restrict__ A, const float* __restrict__ D,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                      const int* __restrict__ slots, TO* __restrict__ out, int channels, int N, int taps) {
  constexpr int NP = NPL * kScanLanes;                      // states a channel's lanes reach, >= N
  constexpr int GROUP = NPL <= 2 ? 8 : NPL <= 4 ? 4 : 2;    // tokens whose independent work the compiler interleaves
  constexpr int BC = kScanChunk * 2 * NP, TOK = kScanChunk * kScanChannels * 4, YS = kScanChunk * kScanChannels;
  constexpr int K = scan_buffers(NPL);
  pdl_wait();
  extern __shared__ __align__(16) float scan_smem[];
  float* bc_s = scan_smem;                                  // [K][chunk][2 NP]: B, then C
  float* tok_s = bc_s + K * BC;                             // [K][chunk][channels of the block][4]: dt, x, z, -
  float* y_s = tok_s + K * TOK;                             // [2][chunk][channels of the block]
  const int e = blockIdx.y, c0 = blockIdx.x * kScanChannels;
  const bool walker = threadIdx.x < kScanWalkers;
  const int tid = walker ? threadIdx.x : threadIdx.x - kScanWalkers;      // place among the walkers, or among the helpers
  const int lane = tid % kScanLanes, ch = tid / kScanLanes;
  const int c = c0 + ch;
  const bool live = c < channels;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0;
  float* slot = state + (size_t)slots[e] * state_stride;
  const int n_chunks = (q_len + kScanChunk - 1) / kScanChunk;

  // helpers: the fetch of chunk j, one group of copies (an empty one behind the last chunk)
  auto stage = [&](int j) {
    if (j >= n_chunks) {
      scan_cp_async_commit();
      return;
    }
    const int base = j * kScanChunk, n_here = min(kScanChunk, q_len - base);
    float* bc = bc_s + (j % K) * BC;
    float* tk = tok_s + (j % K) * TOK;
    for (int idx = tid; idx < kScanChunk * 2 * NP; idx += kScanWalkers) {
      const int i = idx / (2 * NP), r = idx - i * 2 * NP, half = r / NP, n = r - half * NP;
      if (i < n_here && n < N) scan_cp_async_4(bc + idx, dbc + (size_t)(t0 + base + i) * ld_dbc + b_off + half * N + n);
      else bc[idx] = 0.f;
    }
    for (int idx = tid; idx < kScanChunk * kScanChannels; idx += kScanWalkers) {
      const int i = idx / kScanChannels, cc = idx - i * kScanChannels;
      float* dst = tk + (size_t)idx * 4;
      if (i < n_here && c0 + cc < channels) {
        const size_t t = (size_t)(t0 + base + i);
        scan_cp_async_4(dst, dt_raw + t * channels + c0 + cc);
        scan_cp_async_4(dst + 1, x + t * channels + c0 + cc);
        scan_cp_async_4(dst + 2, xz + t * ld_xz + channels + c0 + cc);
      } else {
        dst[0] = dst[1] = dst[2] = 0.f;
      }
    }
    scan_cp_async_commit();
  };
  // helpers: the step sizes of chunk j, once it has landed (a helper's own copies: no barrier between); `behind`
  // groups were committed after the chunk's own
  auto prepare = [&](int j, auto behind) {
    const int n_here = min(kScanChunk, q_len - j * kScanChunk);
    float* tk = tok_s + (j % K) * TOK;
    scan_cp_async_wait<decltype(behind)::value>();
    for (int idx = tid; idx < kScanChunk * kScanChannels; idx += kScanWalkers) {
      const int i = idx / kScanChannels, cc = idx - i * kScanChannels;
      if (i < n_here && c0 + cc < channels) tk[idx * 4] = softplus_f(tk[idx * 4] + (dt_bias ? dt_bias[c0 + cc] : 0.f));
    }
  };
  // helpers: y of chunk j, gated and written: out = (y + D x) * silu(z)
  auto finish = [&](int j) {
    const int base = j * kScanChunk, n_here = min(kScanChunk, q_len - base);
    const float* tk = tok_s + (j % K) * TOK;
    const float* ys = y_s + (j & 1) * YS;
    for (int idx = tid; idx < n_here * kScanChannels; idx += kScanWalkers) {
      const int i = idx / kScanChannels, cc = idx - i * kScanChannels;
      if (c0 + cc < channels) {
        const float xv = tk[idx * 4 + 1], z = tk[idx * 4 + 2];
        out[(size_t)(t0 + base + i) * channels + c0 + cc] = from_float<TO>((ys[idx] + D[c0 + cc] * xv) * silu_f(z));
      }
    }
  };

  float S[NPL], a[NPL];                                     // a lane's states are neighbours: n = lane * NPL + k
  if (walker) {
#pragma unroll
    for (int k = 0; k < NPL; ++k) {
      const int n = lane * NPL + k;
      const bool on = live && n < N;
      S[k] = on ? slot[(size_t)c * N + n] : 0.f;
      a[k] = on ? A[(size_t)c * N + n] * kLog2e : 0.f;      // exp(dt A) = 2^(dt A log2 e)
    }
  } else if (n_chunks > 0) {
    for (int j = 0; j < K - 1; ++j) stage(j);
    prepare(0, std::integral_constant<int, K - 2>());
  }
  for (int j = 0; j < n_chunks; ++j) {
    __syncthreads();       // chunk j lies prepared; the walk over chunk j - 1 is over and its y lies in its buffer
    if (!walker) {
      if (j + 1 < n_chunks) prepare(j + 1, std::integral_constant<int, K - 3>());
      if (j > 0) finish(j - 1);
      stage(j + K - 1);                                     // into the buffer of chunk j - 1
      continue;
    }
    const int n_here = min(kScanChunk, q_len - j * kScanChunk);
    const float* bc = bc_s + (j % K) * BC;
    const float* tk = tok_s + (j % K) * TOK;
    float* ys = y_s + (j & 1) * YS;
#pragma unroll 1
    for (int i0 = 0; i0 < n_here; i0 += GROUP) {
      float y[GROUP];
#pragma unroll
      for (int u = 0; u < GROUP; ++u) {
        const int i = i0 + u;
        const float4 v = *reinterpret_cast<const float4*>(tk + (size_t)(i * kScanChannels + ch) * 4);
        const float dt = v.x, dtx = v.x * v.y;
        float Bv[NPL], Cv[NPL];
        scan_load_row<NPL>(bc + i * 2 * NP + lane * NPL, Bv);
        scan_load_row<NPL>(bc + i * 2 * NP + NP + lane * NPL, Cv);
        y[u] = 0.f;
#pragma unroll
        for (int k = 0; k < NPL; ++k) {
          S[k] = fmaf(scan_exp2(dt * a[k]), S[k], dtx * Bv[k]);
          y[u] = fmaf(S[k], Cv[k], y[u]);
        }
      }
      // the lanes' partial sums of GROUP tokens, added across the 8 lanes: each round a lane hands half of what it
      // holds to its partner and keeps the other half, so 8 tokens cost 4 + 2 + 1 exchanges, and lane l ends with
      // token l's sum; a group of fewer tokens ends with plain rounds (both partners then hold the sum)
      int held = GROUP, tok = 0;
#pragma unroll
      for (int o = kScanLanes / 2; o > 0; o >>= 1) {
        if (held > 1) {
          const int h = held / 2;
          const bool upper = (lane & o) != 0;
#pragma unroll
          for (int u = 0; u < GROUP / 2; ++u)
            if (u < h) {
              const float send = upper ? y[u] : y[u + h], keep = upper ? y[u + h] : y[u];
              y[u] = keep + __shfl_xor_sync(0xffffffffu, send, o);
            }
          tok += upper ? h : 0;
          held = h;
        } else {
          y[0] += __shfl_xor_sync(0xffffffffu, y[0], o);
        }
      }
      if ((lane & (kScanLanes / GROUP - 1)) == 0) ys[(i0 + tok) * kScanChannels + ch] = y[0];
    }
  }
  pdl_trigger();             // a long walk: the kernel behind would only sit on the SMs meanwhile
  __syncthreads();
  if (!walker) {
    if (n_chunks > 0) finish(n_chunks - 1);
    return;
  }
#pragma unroll
  for (int k = 0; k < NPL; ++k) {
    const int n = lane * NPL + k;
    if (live && n < N) slot[(size_t)c * N + n] = S[k];
  }
  // the carried inputs: the last taps - 1 inputs of the channel, of this step or, for a short one, shifted up
  if (live && lane == 0 && taps > 1) {
    float* carry = slot + (size_t)channels * N + (size_t)c * (taps - 1);
    for (int j = 0; j < taps - 1; ++j) {
      const int i = q_len - (taps - 1) + j;                 // place in the entry of the input that lands in carry[j]
      carry[j] = i >= 0 ? xz[(size_t)(t0 + i) * ld_xz + c] : carry[j + q_len];     // reads ahead of what it has written
    }
  }
}

// out = (wa * a / sqrt(mean(a^2) + eps) + wb * b / sqrt(mean(b^2) + eps)) / 2: two sublayers that read the same input,
// each result normed with its own weight, averaged.  One block per token; sums in float32 in an order fixed by the width
// and the block's size.  V elements a thread and access (V = 4 where rows and pointers allow 16 bytes of float32); a
// thread keeps its first PER accesses of a and b in registers for the second pass and reads the rest again.
template <typename TI, typename TO, int V, int PER>
__global__ void paired_rmsnorm_mean_kernel(const TI* __restrict__ a, const float* __restrict__ wa, const TI* __restrict__ b,
                                           const float* __restrict__ wb, float eps, TO* __restrict__ out, int H) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  const int step = blockDim.x * V;
  float ua[PER][V], ub[PER][V];
  float sa = 0.f, sb = 0.f;
  auto fetch = [&](int i, float (&u)[V], float (&v)[V]) {
    if constexpr (V == 4 && sizeof(TI) == 4) {
      const float4 f = *reinterpret_cast<const float4*>(a + base + i), g = *reinterpret_cast<const float4*>(b + base + i);
      u[0] = f.x, u[1] = f.y, u[2] = f.z, u[3] = f.w;
      v[0] = g.x, v[1] = g.y, v[2] = g.z, v[3] = g.w;
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) u[k] = to_float(a[base + i + k]), v[k] = to_float(b[base + i + k]);
    }
  };
  int r = 0;
  for (int i = threadIdx.x * V; i < H; i += step, ++r) {
    float u[V], v[V];
    fetch(i, u, v);
#pragma unroll
    for (int k = 0; k < V; ++k) sa = fmaf(u[k], u[k], sa), sb = fmaf(v[k], v[k], sb);
#pragma unroll
    for (int p = 0; p < PER; ++p)
      if (p == r) {
#pragma unroll
        for (int k = 0; k < V; ++k) ua[p][k] = u[k], ub[p][k] = v[k];
      }
  }
  const float ia = 1.0f / sqrtf(block_sum(sa, scratch) / (float)H + eps);
  const float ib = 1.0f / sqrtf(block_sum(sb, scratch) / (float)H + eps);
  r = 0;
  for (int i = threadIdx.x * V; i < H; i += step, ++r) {
    float u[V], v[V];
    bool kept = false;
#pragma unroll
    for (int p = 0; p < PER; ++p)
      if (p == r) {
        kept = true;
#pragma unroll
        for (int k = 0; k < V; ++k) u[k] = ua[p][k], v[k] = ub[p][k];
      }
    if (!kept) fetch(i, u, v);
#pragma unroll
    for (int k = 0; k < V; ++k)
      out[base + i + k] = from_float<TO>(0.5f * (u[k] * ia * wa[i + k] + v[k] * ib * wb[i + k]));
  }
}

}  // namespace srlm

using namespace srlm;

// xz float32 [T, ld >= channels]: the inputs of the convolution in its first `channels` columns.  conv_w float32
// [channels, taps] (last column: the current token's), conv_b float32 [channels] or null.  state float32
// [slots, state_stride]: per slot channels * N of S, then channels * (taps - 1) carried inputs (read here, renewed by
// srlm_selective_scan).  x_out float32 [T, channels]; x_low [T, channels] in low_dtype, or null.
extern "C" int srlm_scan_conv(const float* xz, long long ld, const float* conv_w, const float* conv_b, const float* state,
                              long long state_stride, const int* entry_of_token, const int* cu_q, const int* slots,
                              float* x_out, void* x_low, int low_dtype, int T, int channels, int N, int taps,
                              cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (channels <= 0 || N <= 0 || taps <= 0 || ld < channels || state_stride < (long long)channels * (N + taps - 1))
    return refuse(ST_BAD_SIZE, "scan_conv: channels=%d N=%d taps=%d ld=%lld state_stride=%lld", channels, N, taps, ld,
                  state_stride);
  // four neighbouring channels a thread where rows and pointers allow 16-byte accesses (the sums are the same)
  const bool wide = channels % 4 == 0 && ld % 4 == 0 && ((uintptr_t)xz | (uintptr_t)x_out | (uintptr_t)x_low) % 16 == 0;
  const long long total = (long long)T * (wide ? channels / 4 : channels);
  const dim3 grid((unsigned)((total + 255) / 256));
  if (wide && taps >= 2 && taps <= 4) {                      // rows read once, weights in registers
    const int run = T >= 512 ? 16 : 4;
    const dim3 rows_grid((channels / 4 + 127) / 128, (T + run - 1) / run);
#define SRLM_CONV_ROWS(TL, TAPS, LOW)                                                                                   \
  launch_pdl(scan_conv_rows_kernel<TL, TAPS>, rows_grid, dim3(128), 0, stream, xz, ld, conv_w, conv_b, state,          \
             state_stride, entry_of_token, cu_q, slots, x_out, LOW, T, channels, N, run)
#define SRLM_CONV_TAPS(TL, LOW)                                  \
  switch (taps) {                                                \
    case 2: SRLM_CONV_ROWS(TL, 2, LOW); break;                   \
    case 3: SRLM_CONV_ROWS(TL, 3, LOW); break;                   \
    default: SRLM_CONV_ROWS(TL, 4, LOW); break;                  \
  }
    if (!x_low) { SRLM_CONV_TAPS(float, (float*)nullptr) }
    else if (low_dtype == DT_BF16) { SRLM_CONV_TAPS(bf16, (bf16*)x_low) }
    else return refuse(ST_BAD_DTYPE, "scan_conv: the second copy of x is bfloat16 (dtype %d)", low_dtype);
#undef SRLM_CONV_TAPS
#undef SRLM_CONV_ROWS
    return launched();
  }
#define SRLM_CONV(TL, V, LOW)                                                                                          \
  launch_pdl(scan_conv_kernel<TL, V>, grid, dim3(256), 0, stream, xz, ld, conv_w, conv_b, state, state_stride,        \
             entry_of_token, cu_q, slots, x_out, LOW, T, channels, N, taps)
  if (!x_low) {
    if (wide) SRLM_CONV(float, 4, (float*)nullptr);
    else SRLM_CONV(float, 1, (float*)nullptr);
  } else if (low_dtype == DT_BF16) {
    if (wide) SRLM_CONV(bf16, 4, (bf16*)x_low);
    else SRLM_CONV(bf16, 1, (bf16*)x_low);
  } else {
    return refuse(ST_BAD_DTYPE, "scan_conv: the second copy of x is bfloat16 (dtype %d)", low_dtype);
  }
#undef SRLM_CONV
  return launched();
}

// x float32 [T, channels] (behind the convolution); xz float32 [T, ld_xz >= 2 channels]: the convolution's inputs, then z;
// dbc float32 [T, ld_dbc]: B in columns [b_off, b_off + N), C in the N columns behind them; dt_raw float32
// [T, channels]; dt_bias, D float32 [channels]; A float32 [channels, N]; out [T, channels] in out_dtype.  max_q_len: the
// most tokens an entry brings (an upper bound will do).
extern "C" int srlm_selective_scan(const float* x, const float* xz, long long ld_xz, const float* dbc, long long ld_dbc,
                                   int b_off, const float* dt_raw, const float* dt_bias, const float* A, const float* D,
                                   float* state, long long state_stride, const int* cu_q, const int* slots, void* out,
                                   int out_dtype, int n_entries, int max_q_len, int channels, int N, int taps,
                                   cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (channels <= 0 || N <= 0 || N > 16 * kScanLanes || taps <= 0 || ld_xz < 2ll * channels || b_off < 0 ||
      ld_dbc < b_off + 2ll * N || state_stride < (long long)channels * (N + taps - 1) || n_entries > 65535)
    return refuse(ST_BAD_SIZE, "selective_scan: channels=%d N=%d (at most %d) taps=%d ld_xz=%lld ld_dbc=%lld b_off=%d "
                  "state_stride=%lld", channels, N, 16 * kScanLanes, taps, ld_xz, ld_dbc, b_off, state_stride);
  const dim3 grid((channels + kScanChannels - 1) / kScanChannels, n_entries);
  int npl = 1;
  while (npl * kScanLanes < N) npl <<= 1;
  const bool early = max_q_len <= 4 * kScanChunk;      // a long walk starts on an empty GPU, its blocks spread evenly
  // some buffers of a chunk's operands (B | C up to the lanes' reach, four words per (token, channel)), two of the block's y
  const size_t smem = (size_t)kScanChunk * (scan_buffers(npl) * (2 * npl * kScanLanes + 4 * kScanChannels) + 2 * kScanChannels) * sizeof(float);
#define SRLM_SCAN(TO, NPL)                                                                                              \
  do {                                                                                                                  \
    static bool sized = false;      /* the widest form asks for more shared memory than a kernel gets unasked */        \
    if (!sized && smem > 48 * 1024) {                                                                                   \
      cudaFuncSetAttribute(selective_scan_kernel<TO, NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      sized = true;                                                                                                     \
    }                                                                                                                   \
    launch_pdl_if(early, selective_scan_kernel<TO, NPL>, grid, dim3(kScanThreads), smem, stream, x, xz, ld_xz, dbc,     \
                  ld_dbc, b_off, dt_raw, dt_bias, A, D, state, state_stride, cu_q, slots, (TO*)out, channels, N, taps); \
  } while (0)
#define SRLM_SCAN_N(TO)                                   \
  switch (npl) {                                          \
    case 1: SRLM_SCAN(TO, 1); break;                      \
    case 2: SRLM_SCAN(TO, 2); break;                      \
    case 4: SRLM_SCAN(TO, 4); break;                      \
    case 8: SRLM_SCAN(TO, 8); break;                      \
    default: SRLM_SCAN(TO, 16);                           \
  }
  if (out_dtype == DT_F32) { SRLM_SCAN_N(float) }
  else if (out_dtype == DT_BF16) { SRLM_SCAN_N(bf16) }
  else return refuse(ST_BAD_DTYPE, "selective_scan: output dtype %d", out_dtype);
#undef SRLM_SCAN_N
#undef SRLM_SCAN
  return launched();
}

// a, b [T, H] in in_dtype; wa, wb float32 [H]; out [T, H] in out_dtype
extern "C" int srlm_paired_rmsnorm_mean(const void* a, const float* wa, const void* b, const float* wb, float eps, void* out,
                                        int in_dtype, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (H <= 0 || !(eps > 0.f) || !wa || !wb) return refuse(ST_BAD_SIZE, "paired_rmsnorm_mean: H=%d eps=%g", H, (double)eps);
  const bool wide = H % 4 == 0 && ((uintptr_t)a | (uintptr_t)b) % 16 == 0;
  const int v = wide ? 4 : 1;
  int block = 64;
  while (block < 1024 && block * 2 * v < H) block <<= 1;      // two accesses a thread, kept in registers between the passes
#define SRLM_PAIRED(TI, TO)                                                                                              \
  do {                                                                                                                   \
    if (wide) launch_pdl(paired_rmsnorm_mean_kernel<TI, TO, 4, 2>, dim3(T), dim3(block), 0, stream, (const TI*)a, wa,    \
                         (const TI*)b, wb, eps, (TO*)out, H);                                                            \
    else launch_pdl(paired_rmsnorm_mean_kernel<TI, TO, 1, 2>, dim3(T), dim3(block), 0, stream, (const TI*)a, wa,         \
                    (const TI*)b, wb, eps, (TO*)out, H);                                                                 \
  } while (0)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) SRLM_PAIRED(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_PAIRED(float, bf16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_PAIRED(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "paired_rmsnorm_mean: input dtype %d with output dtype %d", in_dtype, out_dtype);
#undef SRLM_PAIRED
  return launched();
}
