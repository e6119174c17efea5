// Kernels of blocks that norm after the sum, and small elementwise companions:
//
//   postnorm_scale_add   x <- w' * (alpha x + delta) / sqrt(mean((alpha x + delta)^2) + eps), w' = w or 1 + w (delta one tensor,
//                        or w1 d1 + w2 d2 for two results that are summed with weights on their way in); the float32
//                        stream is rewritten in place and, optionally, copied in the activation dtype for the next
//                        sublayer's products (one kernel, one pass over the row, which stays in shared memory)
//   rmsnorm_columns      RMS norm of a range of columns of a float32 row-major tensor (a latent inside a stacked projection)
//   activation           gelu (exact, erf) or gelu (tanh form) of a range of columns, with an optional bias ahead of it
//   weighted_sum         out = wa a + wb b
//
// All arithmetic float32; sums over a row in an order fixed by the width.
#include "common.cuh"

namespace srlm {

__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

template <typename TD, typename TO>
__global__ void postnorm_scale_add_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                          const TD* __restrict__ delta2, float w1, float w2,
                                          const float* __restrict__ weight, float alpha, float eps, int unit_offset,
                                          TO* __restrict__ out, int H) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float add = delta ? to_float(delta[base + i]) : 0.f;
    if (delta2) add = fmaf(w2, to_float(delta2[base + i]), w1 * add);
    const float v = fmaf(alpha, residual[base + i], add);
    row[i] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
  const float off = unit_offset ? 1.f : 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float y = row[i] * inv * (weight[i] + off);
    residual[base + i] = y;
    if (out) out[base + i] = from_float<TO>(y);
  }
}

template <typename TO>
__global__ void rmsnorm_columns_kernel(const float* __restrict__ in, long long ld, const float* __restrict__ weight,
                                       float eps, int unit_offset, TO* __restrict__ out, int W) {
  pdl_wait();
  pdl_trigger();
  __shared__ float scratch[32];
  const float* p = in + (size_t)blockIdx.x * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) ss += p[i] * p[i];
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  const float off = unit_offset ? 1.f : 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(size_t)blockIdx.x * W + i] = from_float<TO>(p[i] * inv * (weight ? weight[i] + off : 1.f));
}

template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ in, long long ld, const float* __restrict__ bias,
                                  TO* __restrict__ out, int F, size_t total, int kind) {
  pdl_wait();
  pdl_trigger();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / F, f = idx - t * F;
    const float z = to_float(in[t * ld + f]) + (bias ? bias[f] : 0.f);
    out[idx] = from_float<TO>(kind == 0 ? gelu_erf_f(z) : gelu_tanh_f(z));
  }
}

template <typename TI, typename TO>
__global__ void weighted_sum_kernel(const TI* __restrict__ a, float wa, const TI* __restrict__ b, float wb,
                                    TO* __restrict__ out, size_t n) {
  pdl_wait();
  pdl_trigger();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<TO>(fmaf(wb, to_float(b[i]), wa * to_float(a[i])));
}

}  // namespace srlm

using namespace srlm;

#define SRLM_TWO_TYPES(da, db, TA_, TB_, ...)                                                          \
  do {                                                                                                 \
    if ((da) == DT_F32 && (db) == DT_F32) { using TA_ = float; using TB_ = float; __VA_ARGS__; }       \
    else if ((da) == DT_F32 && (db) == DT_BF16) { using TA_ = float; using TB_ = bf16; __VA_ARGS__; }  \
    else if ((da) == DT_BF16 && (db) == DT_F32) { using TA_ = bf16; using TB_ = float; __VA_ARGS__; }  \
    else if ((da) == DT_BF16 && (db) == DT_BF16) { using TA_ = bf16; using TB_ = bf16; __VA_ARGS__; }  \
    else return refuse(ST_BAD_DTYPE, "dtype codes %d, %d are not known", (int)(da), (int)(db));        \
  } while (0)

// residual float32 [T, H] in place; delta [T, H] (delta_dtype) or null; delta2 [T, H] (delta_dtype) or null: then the addend
// is w1 delta + w2 delta2; out [T, H] (out_dtype) or null
extern "C" int srlm_postnorm_scale_add(float* residual, const void* delta, const void* delta2, float w1, float w2,
                                       int delta_dtype, const float* weight, float alpha, float eps, int unit_offset,
                                       void* out, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const size_t smem = (size_t)H * sizeof(float);
  if (H <= 0 || smem > 160 * 1024 || !(eps > 0.f) || (delta2 && !delta))
    return refuse(ST_BAD_SIZE, "postnorm_scale_add: H=%d eps=%g", H, eps);
  const int threads = H >= 2048 ? 512 : 256;
#define SRLM_POSTNORM(TD, TO)                                                                                    \
  do {                                                                                                           \
    auto kern = postnorm_scale_add_kernel<TD, TO>;                                                               \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_pdl(kern, dim3(T), dim3(threads), smem, stream, residual, (const TD*)delta, (const TD*)delta2, w1, w2, \
               weight, alpha, eps, unit_offset, (TO*)out, H);                                                    \
  } while (0)
  SRLM_TWO_TYPES(delta ? delta_dtype : DT_F32, out ? out_dtype : DT_F32, TD, TO, SRLM_POSTNORM(TD, TO));
#undef SRLM_POSTNORM
  return launched();
}

// in float32 [T, ld], the W columns from `in`; weight float32 [W] or null (no weight); out [T, W]
extern "C" int srlm_rmsnorm_columns(const float* in, long long ld, const float* weight, float eps, int unit_offset,
                                    void* out, int out_dtype, int T, int W, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (W <= 0 || ld < W || !(eps > 0.f)) return refuse(ST_BAD_SIZE, "rmsnorm_columns: W=%d ld=%lld", W, ld);
  SRLM_DISPATCH_ACT(out_dtype, TO, launch_pdl(rmsnorm_columns_kernel<TO>, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, stream,
                                              in, ld, weight, eps, unit_offset, (TO*)out, W));
  return launched();
}

// in [T, ld] (in_dtype), the F columns from `in`; bias float32 [F] or null; out [T, F]; kind 0: gelu with erf, 1: its tanh form
extern "C" int srlm_activation(const void* in, int in_dtype, long long ld, const float* bias, void* out, int out_dtype,
                               int T, int F, int kind, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (F <= 0 || ld < F || kind < 0 || kind > 1) return refuse(ST_BAD_SIZE, "activation: F=%d ld=%lld kind=%d", F, ld, kind);
  const size_t total = (size_t)T * F;
  const unsigned grid = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  SRLM_TWO_TYPES(in_dtype, out_dtype, TI, TO, launch_pdl(activation_kernel<TI, TO>, dim3(grid), dim3(256), 0, stream,
                                                         (const TI*)in, ld, bias, (TO*)out, F, total, kind));
  return launched();
}

extern "C" int srlm_weighted_sum(const void* a, float wa, const void* b, float wb, int in_dtype, void* out, int out_dtype,
                                 long long n, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  const unsigned grid = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  SRLM_TWO_TYPES(in_dtype, out_dtype, TI, TO, launch_pdl(weighted_sum_kernel<TI, TO>, dim3(grid), dim3(256), 0, stream,
                                                         (const TI*)a, wa, (const TI*)b, wb, (TO*)out, (size_t)n));
  return launched();
}
