// A short causal convolution over time, per channel, for the ragged batch of a step:
//
//   y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c] (+ bias),   u = 0 before a request's first token
//
// The inputs u of a step are C columns of a float32 row-major tensor (a projection's result), optionally plus a bias per
// channel.  The taps - 1 inputs ahead of a portion's first token come from the request's slot, where the carry kernel
// leaves the last taps - 1 inputs of every channel after each step ([taps - 1][C] floats at state_off of the slot's row,
// oldest first; zeros for a new request).  So a request may be cut anywhere, down to single tokens.
//
//   short_conv             y as float32 (and, optionally, a copy in the activation dtype)
//   conv_carry             renews the slots' carried inputs; runs behind every kernel that reads them
//   conv_norm_rope_append  for an attention whose q, k and v each pass such a convolution: convolution, RMS norm per head
//                          of q and k, rotation of their leading pairs, q to its buffer and k, v to the pages, in one kernel
#include "common.cuh"

namespace srlm {

constexpr int kMaxTaps = 16;

struct ConvInput {
  const float* proj;        // [T, ld], the channels' columns start at proj
  long long ld;
  const float* in_bias;     // [C] or null: added to every input of the step (the carried ones hold it already)
  const float* state;       // [slots, state_stride]
  long long state_stride;
  int state_off;
  int taps, C;
};

// The convolution of channel c at token t, which is token `idx` of its entry's portion.
__device__ __forceinline__ float conv_at(const ConvInput& in, const float* __restrict__ w, int t, int idx, int slot, int c) {
  float acc = 0.f;
  const float bias = in.in_bias ? in.in_bias[c] : 0.f;
  for (int j = 0; j < in.taps; ++j) {
    const int back = in.taps - 1 - j;
    float u;
    if (back <= idx) u = in.proj[(size_t)(t - back) * in.ld + c] + bias;
    else u = in.state[(size_t)slot * in.state_stride + in.state_off + (size_t)(in.taps - 1 - (back - idx)) * in.C + c];
    acc = fmaf(w[(size_t)c * in.taps + j], u, acc);
  }
  return acc;
}

template <typename TO>
__global__ void short_conv_kernel(ConvInput in, const float* __restrict__ w, const float* __restrict__ out_bias,
                                  const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, float* __restrict__ out, TO* __restrict__ out_low, int T) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.y;
  const int e = entry_of_token[t];
  const int idx = t - cu_q[e], slot = slots[e];
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < in.C; c += gridDim.x * blockDim.x) {
    const float y = conv_at(in, w, t, idx, slot, c) + (out_bias ? out_bias[c] : 0.f);
    out[(size_t)t * in.C + c] = y;
    if (out_low) out_low[(size_t)t * in.C + c] = from_float<TO>(y);
  }
}

// New carry of entry e: the last taps - 1 of (old carry, the portion's inputs).
__global__ void conv_carry_kernel(ConvInput in, float* __restrict__ state, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots) {
  pdl_wait();
  pdl_trigger();
  const int e = blockIdx.y;
  const int first = cu_q[e], n = cu_q[e + 1] - first;
  const int keep = in.taps - 1;
  float* carry = state + (size_t)slots[e] * in.state_stride + in.state_off;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < in.C; c += gridDim.x * blockDim.x) {
    float fresh[kMaxTaps];
    const float bias = in.in_bias ? in.in_bias[c] : 0.f;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k >= keep) break;
      const int j = n - keep + k;                          // which token of the portion lands in place k
      fresh[k] = j >= 0 ? in.proj[(size_t)(first + j) * in.ld + c] + bias : carry[(size_t)(k + n) * in.C + c];
    }
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k >= keep) break;
      carry[(size_t)k * in.C + c] = fresh[k];
    }
  }
}

// One warp per (token, head) of the stacked projection [q heads | k heads | v heads]; the conv weights are stacked the
// same way.  Rotation: the first 2 * pairs elements of a q or k head, partners (i, i + pairs) or (2i, 2i + 1).
template <typename TQ, typename TC>
__global__ void conv_norm_rope_append_kernel(ConvInput in, const float* __restrict__ w, const float* __restrict__ q_norm_w,
                                             const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                                             const float* __restrict__ sin_t, int pairs, int interleaved,
                                             const int* __restrict__ entry_of_token, const int* __restrict__ cu_q,
                                             const int* __restrict__ slots, const int* __restrict__ kv_slot,
                                             TQ* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                             int T, int nq, int nkv, int dk, int dv, int page_size) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float head_smem[];                      // a head per warp
  const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
  const int heads_total = nq + 2 * nkv;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
  if (warp >= (long long)T * heads_total) return;
  const int t = (int)(warp / heads_total), head = (int)(warp % heads_total);
  const int e = entry_of_token[t];
  const int idx = t - cu_q[e], slot = slots[e];
  const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
  const int d = (is_q || is_k) ? dk : dv;
  const int c0 = is_q ? head * dk : is_k ? nq * dk + (head - nq) * dk : (nq + nkv) * dk + (head - nq - nkv) * dv;
  float* x = head_smem + (size_t)warp_in_block * (dk > dv ? dk : dv);
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float y = conv_at(in, w, t, idx, slot, c0 + i);
    x[i] = y;
    ss += y * y;
  }
  __syncwarp();
  if (is_q || is_k) {
    const float* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
      for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * nw[i];
      __syncwarp();
    }
  }
  const int row = kv_slot ? kv_slot[t] : -1;
  for (int i = lane; i < d; i += 32) {
    float v = x[i];
    if ((is_q || is_k) && i < 2 * pairs) {
      const int p = interleaved ? (i >> 1) : (i < pairs ? i : i - pairs);
      const bool second = interleaved ? (i & 1) : (i >= pairs);
      const float other = x[interleaved ? (i ^ 1) : (second ? i - pairs : i + pairs)];
      const float c = cos_t[(size_t)t * pairs + p], s = sin_t[(size_t)t * pairs + p];
      v = second ? v * c + other * s : v * c - other * s;
    }
    if (is_q) {
      q_out[(size_t)t * nq * dk + (size_t)head * dk + i] = from_float<TQ>(v);
    } else if (row >= 0) {
      const int page = row / page_size, at = row % page_size;
      if (is_k) k_cache[(((size_t)page * nkv + (head - nq)) * page_size + at) * dk + i] = from_float<TC>(v);
      else v_cache[(((size_t)page * nkv + (head - nq - nkv)) * page_size + at) * dv + i] = from_float<TC>(v);
    }
  }
}

}  // namespace srlm

using namespace srlm;

static int conv_input_ok(const char* what, int taps, int C, long long ld, long long state_stride, int state_off) {
  if (taps < 1 || taps > kMaxTaps || C <= 0 || ld < C || state_off < 0 ||
      (taps > 1 && state_stride < state_off + (long long)(taps - 1) * C))
    return refuse(ST_BAD_SIZE, "%s: taps=%d (1..%d) channels=%d ld=%lld state row %lld from %d", what, taps, kMaxTaps, C, ld,
                  state_stride, state_off);
  return ST_OK;
}

// proj float32 [T, ld] (the channels' first column at proj); w float32 [C, taps]; out float32 [T, C]; out_low [T, C] or null
extern "C" int srlm_short_conv(const float* proj, long long ld, const float* in_bias, const float* w, const float* out_bias,
                               const float* state, long long state_stride, int state_off, const int* entry_of_token,
                               const int* cu_q, const int* slots, float* out, void* out_low, int low_dtype, int T, int C,
                               int taps, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (int r = conv_input_ok("short_conv", taps, C, ld, state_stride, state_off)) return r;
  ConvInput in{proj, ld, in_bias, state, state_stride, state_off, taps, C};
  dim3 grid((unsigned)((C + 255) / 256), (unsigned)T);
  if (T > 65535) return refuse(ST_BAD_SIZE, "short_conv: %d tokens", T);
  SRLM_DISPATCH_ACT(out_low ? low_dtype : DT_F32, TO,
                    launch_pdl(short_conv_kernel<TO>, grid, dim3(256), 0, stream, in, w, out_bias, entry_of_token, cu_q,
                               slots, out, (TO*)out_low, T));
  return launched();
}

extern "C" int srlm_conv_carry(const float* proj, long long ld, const float* in_bias, float* state, long long state_stride,
                               int state_off, const int* cu_q, const int* slots, int n_entries, int C, int taps,
                               cudaStream_t stream) {
  if (n_entries <= 0 || taps <= 1) return ST_OK;
  if (int r = conv_input_ok("conv_carry", taps, C, ld, state_stride, state_off)) return r;
  if (n_entries > 65535) return refuse(ST_BAD_SIZE, "conv_carry: %d entries", n_entries);
  ConvInput in{proj, ld, in_bias, state, state_stride, state_off, taps, C};
  launch_pdl(conv_carry_kernel, dim3((unsigned)((C + 255) / 256), (unsigned)n_entries), dim3(256), 0, stream, in, state,
             cu_q, slots);
  return launched();
}

// proj float32 [T, ld]: q heads (nq dk) | k heads (nkv dk) | v heads (nkv dv); w float32 [channels, taps] stacked alike;
// q_norm_w / k_norm_w float32 [dk] or null; q_out [T, nq dk] (q_dtype); pages [page, kv head, token in page, size]
extern "C" int srlm_conv_norm_rope_append(const float* proj, long long ld, const float* w, const float* state,
                                          long long state_stride, int state_off, const float* q_norm_w,
                                          const float* k_norm_w, float eps, const float* cos_t, const float* sin_t,
                                          int pairs, int interleaved, const int* entry_of_token, const int* cu_q,
                                          const int* slots, const int* kv_slot, void* q_out, int q_dtype, void* k_cache,
                                          void* v_cache, int cache_dtype, int T, int nq, int nkv, int dk, int dv,
                                          int page_size, int taps, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const int C = nq * dk + nkv * (dk + dv);
  if (nq <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || pairs < 0 || 2 * pairs > dk ||
      (pairs > 0 && (!cos_t || !sin_t)) || ((q_norm_w || k_norm_w) && !(eps > 0.f)))
    return refuse(ST_BAD_SIZE, "conv_norm_rope_append: nq=%d nkv=%d dk=%d dv=%d pairs=%d", nq, nkv, dk, dv, pairs);
  if (int r = conv_input_ok("conv_norm_rope_append", taps, C, ld, state_stride, state_off)) return r;
  ConvInput in{proj, ld, nullptr, state, state_stride, state_off, taps, C};
  const int warps = 4;
  const size_t smem = (size_t)warps * (dk > dv ? dk : dv) * sizeof(float);
  if (smem > 48 * 1024) return refuse(ST_BAD_SIZE, "conv_norm_rope_append: heads of %d elements", dk > dv ? dk : dv);
  const long long total = (long long)T * (nq + 2 * nkv);
  const unsigned grid = (unsigned)((total + warps - 1) / warps);
#define SRLM_CNRA(TQ, TC)                                                                                              \
  launch_pdl(conv_norm_rope_append_kernel<TQ, TC>, dim3(grid), dim3(warps * 32), smem, stream, in, w, q_norm_w, k_norm_w, \
             eps, cos_t, sin_t, pairs, interleaved, entry_of_token, cu_q, slots, kv_slot, (TQ*)q_out, (TC*)k_cache,     \
             (TC*)v_cache, T, nq, nkv, dk, dv, page_size)
  if (q_dtype == DT_F32 && cache_dtype == DT_F32) SRLM_CNRA(float, float);
  else if (q_dtype == DT_F32 && cache_dtype == DT_BF16) SRLM_CNRA(float, bf16);
  else if (q_dtype == DT_BF16 && cache_dtype == DT_BF16) SRLM_CNRA(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "conv_norm_rope_append: q dtype %d with cache dtype %d", q_dtype, cache_dtype);
#undef SRLM_CNRA
  return launched();
}
