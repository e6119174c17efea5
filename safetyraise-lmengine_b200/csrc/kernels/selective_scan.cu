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
//   conv   one thread per (token, channel): reads the step's inputs, and the slot's carried inputs for the first
//          taps - 1 tokens of an entry
//   scan   one block per (entry, 16 channels): 8 lanes share a channel's N states and walk the entry's tokens in
//          order, staged through shared memory in chunks; then the block renews the slot's S and carried inputs.
//          A channel's sums do not depend on what else is in the step or on how the tokens were cut into steps.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// state of a slot: [channels * N] S, then [channels * (taps - 1)] carried inputs, oldest first
template <typename TL>
__global__ void scan_conv_kernel(const float* __restrict__ xz, long long ld, const float* __restrict__ conv_w,
                                 const float* __restrict__ conv_b, const float* __restrict__ state, long long state_stride,
                                 const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                                 const int* __restrict__ slots, float* __restrict__ x_out, TL* __restrict__ x_low,
                                 int T, int channels, int N, int taps) {
  pdl_wait();
  pdl_trigger();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * channels) return;
  const int t = (int)(idx / channels), c = (int)(idx - (long long)t * channels);
  const int e = entry_of_token[t];
  const int i = t - cu_q[e];                               // the token's place in its entry
  const float* carry = state + (size_t)slots[e] * state_stride + (size_t)channels * N + (size_t)c * (taps - 1);
  float acc = conv_b ? conv_b[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;                         // tap j weighs the input `back` tokens ago
    const float v = back <= i ? xz[(size_t)(t - back) * ld + c] : carry[taps - 1 + i - back];
    acc = fmaf(conv_w[(size_t)c * taps + j], v, acc);
  }
  const float y = silu_f(acc);
  x_out[idx] = y;
  if (x_low) x_low[idx] = from_float<TL>(y);
}

constexpr int kScanLanes = 8, kScanChannels = 16, kScanChunk = 16;

template <typename TO, int NPL>
__global__ void __launch_bounds__(kScanLanes* kScanChannels)
selective_scan_kernel(const float* __restrict__ x, const float* __restrict__ xz, long long ld_xz,
                      const float* __restrict__ dbc, long long ld_dbc, int b_off, const float* __restrict__ dt_raw,
                      const float* __restrict__ dt_bias, const float* __restrict__ A, const float* __restrict__ D,
                      float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                      const int* __restrict__ slots, TO* __restrict__ out, int channels, int N, int taps) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float scan_smem[];
  float* bc_s = scan_smem;                                  // [chunk][2 N]: B, then C
  float* tok_s = bc_s + kScanChunk * 2 * N;                 // [chunk][channels of the block][3]: dt, x, z
  const int e = blockIdx.y, c0 = blockIdx.x * kScanChannels;
  const int tid = threadIdx.x, lane = tid % kScanLanes, ch = tid / kScanLanes;
  const int c = c0 + ch;
  const bool live = c < channels;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0;
  float* slot = state + (size_t)slots[e] * state_stride;
  float S[NPL], a[NPL];
#pragma unroll
  for (int k = 0; k < NPL; ++k) {
    const int n = lane + k * kScanLanes;
    const bool on = live && n < N;
    S[k] = on ? slot[(size_t)c * N + n] : 0.f;
    a[k] = on ? A[(size_t)c * N + n] : 0.f;
  }
  const float d_c = live ? D[c] : 0.f;
  for (int base = 0; base < q_len; base += kScanChunk) {
    const int n_here = min(kScanChunk, q_len - base);
    __syncthreads();                                        // the chunk before is no longer read
    for (int idx = tid; idx < n_here * 2 * N; idx += blockDim.x) {
      const int i = idx / (2 * N), n = idx - i * 2 * N;
      bc_s[i * 2 * N + n] = dbc[(size_t)(t0 + base + i) * ld_dbc + b_off + n];
    }
    for (int idx = tid; idx < n_here * kScanChannels; idx += blockDim.x) {
      const int i = idx / kScanChannels, cc = idx - i * kScanChannels;
      const size_t t = (size_t)(t0 + base + i);
      const bool on = c0 + cc < channels;
      float* dst = tok_s + (size_t)(i * kScanChannels + cc) * 3;
      dst[0] = on ? softplus_f(dt_raw[t * channels + c0 + cc] + (dt_bias ? dt_bias[c0 + cc] : 0.f)) : 0.f;
      dst[1] = on ? x[t * channels + c0 + cc] : 0.f;
      dst[2] = on ? xz[t * ld_xz + channels + c0 + cc] : 0.f;
    }
    __syncthreads();
    for (int i = 0; i < n_here; ++i) {
      const float* tk = tok_s + (size_t)(i * kScanChannels + ch) * 3;
      const float dt = tk[0], xv = tk[1], z = tk[2];
      const float dtx = dt * xv;
      const float* Bt = bc_s + i * 2 * N;
      float y = 0.f;
#pragma unroll
      for (int k = 0; k < NPL; ++k) {
        const int n = lane + k * kScanLanes;
        if (n < N) {
          S[k] = fmaf(expf(dt * a[k]), S[k], dtx * Bt[n]);
          y = fmaf(S[k], Bt[N + n], y);
        }
      }
#pragma unroll
      for (int o = kScanLanes / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (lane == 0 && live) out[(size_t)(t0 + base + i) * channels + c] = from_float<TO>((y + d_c * xv) * silu_f(z));
    }
  }
#pragma unroll
  for (int k = 0; k < NPL; ++k) {
    const int n = lane + k * kScanLanes;
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
// each result normed with its own weight, averaged.  One block per token; sums in float32 in an order fixed by the width.
template <typename TI, typename TO>
__global__ void paired_rmsnorm_mean_kernel(const TI* __restrict__ a, const float* __restrict__ wa, const TI* __restrict__ b,
                                           const float* __restrict__ wb, float eps, TO* __restrict__ out, int H) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float u = to_float(a[base + i]), v = to_float(b[base + i]);
    sa += u * u;
    sb += v * v;
  }
  const float ia = 1.0f / sqrtf(block_sum(sa, scratch) / (float)H + eps);
  const float ib = 1.0f / sqrtf(block_sum(sb, scratch) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[base + i] = from_float<TO>(0.5f * (to_float(a[base + i]) * ia * wa[i] + to_float(b[base + i]) * ib * wb[i]));
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
  const long long total = (long long)T * channels;
  const dim3 grid((unsigned)((total + 255) / 256));
  if (!x_low)
    launch_pdl(scan_conv_kernel<float>, grid, dim3(256), 0, stream, xz, ld, conv_w, conv_b, state, state_stride,
               entry_of_token, cu_q, slots, x_out, (float*)nullptr, T, channels, N, taps);
  else if (low_dtype == DT_BF16)
    launch_pdl(scan_conv_kernel<bf16>, grid, dim3(256), 0, stream, xz, ld, conv_w, conv_b, state, state_stride,
               entry_of_token, cu_q, slots, x_out, (bf16*)x_low, T, channels, N, taps);
  else
    return refuse(ST_BAD_DTYPE, "scan_conv: the second copy of x is bfloat16 (dtype %d)", low_dtype);
  return launched();
}

// x float32 [T, channels] (behind the convolution); xz float32 [T, ld_xz >= 2 channels]: the convolution's inputs, then z;
// dbc float32 [T, ld_dbc]: B in columns [b_off, b_off + N), C in the N columns behind them; dt_raw float32
// [T, channels]; dt_bias, D float32 [channels]; A float32 [channels, N]; out [T, channels] in out_dtype.
extern "C" int srlm_selective_scan(const float* x, const float* xz, long long ld_xz, const float* dbc, long long ld_dbc,
                                   int b_off, const float* dt_raw, const float* dt_bias, const float* A, const float* D,
                                   float* state, long long state_stride, const int* cu_q, const int* slots, void* out,
                                   int out_dtype, int n_entries, int channels, int N, int taps, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (channels <= 0 || N <= 0 || N > 16 * kScanLanes || taps <= 0 || ld_xz < 2ll * channels || b_off < 0 ||
      ld_dbc < b_off + 2ll * N || state_stride < (long long)channels * (N + taps - 1) || n_entries > 65535)
    return refuse(ST_BAD_SIZE, "selective_scan: channels=%d N=%d (at most %d) taps=%d ld_xz=%lld ld_dbc=%lld b_off=%d "
                  "state_stride=%lld", channels, N, 16 * kScanLanes, taps, ld_xz, ld_dbc, b_off, state_stride);
  const dim3 grid((channels + kScanChannels - 1) / kScanChannels, n_entries);
  const size_t smem = (size_t)kScanChunk * (2 * N + 3 * kScanChannels) * sizeof(float);
  int npl = 1;
  while (npl * kScanLanes < N) npl <<= 1;
#define SRLM_SCAN(TO, NPL)                                                                                              \
  launch_pdl(selective_scan_kernel<TO, NPL>, grid, dim3(kScanLanes * kScanChannels), smem, stream, x, xz, ld_xz, dbc, ld_dbc, \
             b_off, dt_raw, dt_bias, A, D, state, state_stride, cu_q, slots, (TO*)out, channels, N, taps)
#define SRLM_SCAN_N(TO)                                   \
  switch (npl) {                                          \
    case 1: SRLM_SCAN(TO, 1); break;                      \
    case 2: SRLM_SCAN(TO, 2); break;                      \
    case 4: SRLM_SCAN(TO, 4); break;                      \
    case 8: SRLM_SCAN(TO, 8); break;                      \
    default: SRLM_SCAN(TO, 16); break;                    \
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
  int block = 64;
  while (block < 1024 && block * 4 < H) block <<= 1;
#define SRLM_PAIRED(TI, TO)                                                                                    \
  launch_pdl(paired_rmsnorm_mean_kernel<TI, TO>, dim3(T), dim3(block), 0, stream, (const TI*)a, wa, (const TI*)b, wb, eps, \
             (TO*)out, H)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) SRLM_PAIRED(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_PAIRED(float, bf16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_PAIRED(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "paired_rmsnorm_mean: input dtype %d with output dtype %d", in_dtype, out_dtype);
#undef SRLM_PAIRED
  return launched();
}
