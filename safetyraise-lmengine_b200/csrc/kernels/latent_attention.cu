// Attention over a cached latent: the pages hold, per token, one vector c of `rank` elements (the
// RMS-normed down projection) followed by one rotated key part of `rot` elements shared by all heads.
// Per head the unrotated key would be U_k c and the value U_v c; neither is ever formed:
//
//   score(i, j) = (q_i . U_k c_j + qr_i . kr_j) * scale = ((U_k^T q_i) . c_j + qr_i . kr_j) * scale
//   out_i       = U_v sum_j p_ij c_j
//
// so the attention itself runs with one KV head whose keys are [c, kr] and whose values are the keys'
// first `rank` elements (paged_attention_general), between the three kernels of this file:
//   latent_append  -- norm of c, rotation of kr, append to the pages;
//   latent_absorb  -- per head [U_k^T q | rotated qr] as float32 queries of size rank + rot;
//   latent_expand  -- per head U_v (sum p c), times the sigmoid of the head's output gate.
// Rotation: element pairs (2i, 2i + 1), or (i, i + pairs) when `halves` is set, i < pairs, by the step's cos / sin
// tables [T, pairs]; the rest of the rotated part passes unchanged.  All arithmetic float32.
#include "common.cuh"

namespace srlm {

// Element i of a rotated part `src` of token t (i < 2 * pairs).
template <typename TP>
__device__ __forceinline__ float rotated_element(const TP* __restrict__ src, int i, size_t t, int pairs, int halves,
                                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t) {
  const int p = halves ? (i < pairs ? i : i - pairs) : (i >> 1);
  const bool second = halves ? i >= pairs : (i & 1);
  const float other = to_float(src[halves ? (second ? i - pairs : i + pairs) : (i ^ 1)]);
  const float c = cos_t[t * pairs + p], s = sin_t[t * pairs + p], v = to_float(src[i]);
  return second ? v * c + other * s : v * c - other * s;
}

constexpr int kTokTile = 16;

// One block per token.  proj row: [.. | c_raw (rank) | kr_raw (rot) | ..] starting at column c_off.  q_out != null: the
// same block also norms the q_width columns from q_col (a latent of the queries in the same stacked projection) with
// q_norm_w into q_out [T, q_width].
template <typename TP, typename TC, typename TQ>
__global__ void latent_append_kernel(const TP* __restrict__ proj, long long ldp, int c_off,
                                     const float* __restrict__ norm_w, float eps, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int pairs, int halves, TC* __restrict__ cache,
                                     const int* __restrict__ kv_slot, int rank, int rot, int q_col, int q_width,
                                     const float* __restrict__ q_norm_w, TQ* __restrict__ q_out) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const TP* p = proj + (size_t)t * ldp + c_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(p[i]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  TC* row = cache + (size_t)kv_slot[t] * (rank + rot);      // one KV head: the flat slot is the row
  for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_float<TC>(to_float(p[i]) * inv * norm_w[i]);
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    const float v = i < 2 * pairs ? rotated_element(p + rank, i, (size_t)t, pairs, halves, cos_t, sin_t) : to_float(p[rank + i]);
    row[rank + i] = from_float<TC>(v);
  }
  if (q_out) {
    const TP* q = proj + (size_t)t * ldp + q_col;
    float qs = 0.f;
    for (int i = threadIdx.x; i < q_width; i += blockDim.x) {
      const float v = to_float(q[i]);
      qs += v * v;
    }
    const float q_inv = 1.0f / sqrtf(block_sum(qs, scratch) / (float)q_width + eps);
    for (int i = threadIdx.x; i < q_width; i += blockDim.x)
      q_out[(size_t)t * q_width + i] = from_float<TQ>(to_float(q[i]) * q_inv * q_norm_w[i]);
  }
}

// The two per-head products: out[t, h, c] = sum_k in[t, h, k] * W[h, k, c].  A block takes 16 tokens, one head
// and 32 columns; its four warps each take a quarter of k (a lane owns a column, so a warp reads 32
// consecutive weights) and their partial sums are added in warp order through shared memory: the order of
// every sum depends on the sizes alone.  Decode steps launch heads x columns / 32 blocks, not one per head.
constexpr int kColTile = 32, kProductWarps = 4;

template <typename TW>
__device__ __forceinline__ void head_product(const float* __restrict__ in_s, int K, const TW* __restrict__ w, int cols,
                                             int col, float* __restrict__ red, float (&sum)[kTokTile / kProductWarps]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per = (K + kProductWarps - 1) / kProductWarps, k0 = warp * per, k1 = min(K, k0 + per);
  float acc[kTokTile];
#pragma unroll
  for (int tt = 0; tt < kTokTile; ++tt) acc[tt] = 0.f;
  if (col < cols) {
    for (int k = k0; k < k1; ++k) {
      const float wv = to_float(w[(size_t)k * cols + col]);
#pragma unroll
      for (int tt = 0; tt < kTokTile; ++tt) acc[tt] += in_s[tt * K + k] * wv;
    }
  }
#pragma unroll
  for (int tt = 0; tt < kTokTile; ++tt) red[(warp * kTokTile + tt) * kColTile + lane] = acc[tt];
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kTokTile / kProductWarps; ++i) {      // this warp finishes four of the sixteen tokens
    const int tt = warp * (kTokTile / kProductWarps) + i;
    float v = 0.f;
#pragma unroll
    for (int ww = 0; ww < kProductWarps; ++ww) v += red[(ww * kTokTile + tt) * kColTile + lane];
    sum[i] = v;
  }
}

// Block (token tile, head, 32 columns of the latent).  q row: heads x [dim unrotated | rot rotated].
// uk: [heads, dim, rank].  q_out: float32 [T, heads, rank + rot]; the blocks of the first columns also rotate.
template <typename TP, typename TW>
__global__ void __launch_bounds__(kProductWarps * 32)
latent_absorb_kernel(const TP* __restrict__ proj, long long ldp, const TW* __restrict__ uk,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pairs, int halves,
                     float* __restrict__ q_out, int T, int heads, int dim, int rot, int rank) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ float sh[];                              // [kTokTile][dim] | [warps][kTokTile][32]
  float* q_s = sh;
  float* red = sh + kTokTile * dim;
  const int t0 = blockIdx.x * kTokTile, h = blockIdx.y;
  const int n = min(kTokTile, T - t0);
  for (int idx = threadIdx.x; idx < kTokTile * dim; idx += blockDim.x) {
    const int tt = idx / dim, d = idx - tt * dim;
    q_s[idx] = tt < n ? to_float(proj[(size_t)(t0 + tt) * ldp + (size_t)h * (dim + rot) + d]) : 0.f;
  }
  __syncthreads();
  const int qd = rank + rot, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.z * kColTile + lane;
  float sum[kTokTile / kProductWarps];
  head_product(q_s, dim, uk + (size_t)h * dim * rank, rank, col, red, sum);
#pragma unroll
  for (int i = 0; i < kTokTile / kProductWarps; ++i) {
    const int tt = warp * (kTokTile / kProductWarps) + i;
    if (tt < n && col < rank) q_out[((size_t)(t0 + tt) * heads + h) * qd + col] = sum[i];
  }
  if (blockIdx.z != 0) return;
  for (int idx = threadIdx.x; idx < n * rot; idx += blockDim.x) {
    const int tt = idx / rot, i = idx - tt * rot, t = t0 + tt;
    const TP* src = proj + (size_t)t * ldp + (size_t)h * (dim + rot) + dim;
    q_out[((size_t)t * heads + h) * qd + rank + i] =
        i < 2 * pairs ? rotated_element(src, i, (size_t)t, pairs, halves, cos_t, sin_t) : to_float(src[i]);
  }
}

// Block (token tile, head, 32 value columns).  o_lat: float32 [T, heads, rank]; uv_t: [heads, rank, dv] (the up
// projection of the values, transposed per head); gate: column g_off + h of the projection row, or none.
template <typename TP, typename TW, typename TA>
__global__ void __launch_bounds__(kProductWarps * 32)
latent_expand_kernel(const float* __restrict__ o_lat, const TW* __restrict__ uv_t, const TP* __restrict__ proj,
                     long long ldp, int g_off, TA* __restrict__ out, int T, int heads, int rank, int dv) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ __align__(16) float sh[];                // [kTokTile][rank] | [warps][kTokTile][32]
  float* o_s = sh;
  float* red = sh + kTokTile * rank;
  const int t0 = blockIdx.x * kTokTile, h = blockIdx.y;
  const int n = min(kTokTile, T - t0);
  if (rank % 4 == 0) {          // 16-byte pieces: a quarter of the trips to memory
    const int r4 = rank / 4;
    for (int idx = threadIdx.x; idx < kTokTile * r4; idx += blockDim.x) {
      const int tt = idx / r4, r = (idx - tt * r4) * 4;
      const float4 v = tt < n ? *reinterpret_cast<const float4*>(o_lat + ((size_t)(t0 + tt) * heads + h) * rank + r)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(o_s + tt * rank + r) = v;
    }
  } else {
    for (int idx = threadIdx.x; idx < kTokTile * rank; idx += blockDim.x) {
      const int tt = idx / rank, r = idx - tt * rank;
      o_s[idx] = tt < n ? o_lat[((size_t)(t0 + tt) * heads + h) * rank + r] : 0.f;
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.z * kColTile + lane;
  float sum[kTokTile / kProductWarps];
  head_product(o_s, rank, uv_t + (size_t)h * rank * dv, dv, col, red, sum);
#pragma unroll
  for (int i = 0; i < kTokTile / kProductWarps; ++i) {
    const int tt = warp * (kTokTile / kProductWarps) + i;
    if (tt >= n || col >= dv) continue;
    float g = 1.f;
    if (g_off >= 0) g = 1.f / (1.f + expf(-to_float(proj[(size_t)(t0 + tt) * ldp + g_off + h])));
    out[((size_t)(t0 + tt) * heads + h) * dv + col] = from_float<TA>(sum[i] * g);
  }
}

// ---- prompts: per-head keys and values formed for the step ----------------------------------------------
// A prompt attends in the heads' own space (dim + rot per key, vdim per value: a third of the latent form's
// arithmetic).  latent_gather copies the latents of every entry's context out of the pages into one
// contiguous matrix, row cu_kv[e] + j for key j of entry e (from the first key that the step's windows still see); one matrix product with [U_k; U_v] then gives all
// heads' unrotated keys and values; the rotated key part stays in the pages and is read from there.
template <typename TC>
__global__ void latent_gather_kernel(const TC* __restrict__ cache, TC* __restrict__ dst,
                                     const int* __restrict__ block_table, int table_stride,
                                     const int* __restrict__ cu_kv, const int* __restrict__ kv_first,
                                     const int* __restrict__ kv_lens, int page_size, int width, int rank) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  // keys kv_first[e] .. kv_lens[e] - 1 of entry e go to the rows cu_kv[e] + j (cu_kv[e] is where key 0 would lie)
  const int e = blockIdx.y;
  const int first = kv_first ? kv_first[e] : 0;
  const int* table = block_table + (size_t)e * table_stride;
  for (int j = first + blockIdx.x; j < kv_lens[e]; j += gridDim.x) {
    const int page = table[j / page_size];                  // negative: a page behind every window, given back
    TC* out = dst + (size_t)(cu_kv[e] + j) * rank;
    const size_t row = (size_t)(page < 0 ? 0 : page) * page_size + (j % page_size);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) out[i] = page < 0 ? from_float<TC>(0.f) : cache[row * width + i];
  }
}

// q_out float32 [T, heads, dim + rot]: the unrotated part as projected, the rest rotated.
template <typename TP>
__global__ void latent_rotate_q_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int pairs, int halves, float* __restrict__ q_out,
                                       int heads, int dim, int rot) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const int t = blockIdx.x, hd = dim + rot;
  for (int idx = threadIdx.x; idx < heads * hd; idx += blockDim.x) {
    const int h = idx / hd, i = idx - h * hd;
    const TP* src = proj + (size_t)t * ldp + (size_t)h * hd;
    const int r = i - dim;
    q_out[(size_t)t * heads * hd + idx] =
        (r >= 0 && r < 2 * pairs) ? rotated_element(src + dim, r, (size_t)t, pairs, halves, cos_t, sin_t) : to_float(src[i]);
  }
}

// out[t, h, :] = in[t, h, :] * sigmoid(proj[t, g_off + h])   (g_off < 0: no gate, a change of type only)
template <typename TI, typename TP, typename TA>
__global__ void head_gate_kernel(const TI* in, const TP* __restrict__ proj, long long ldp, int g_off,
                                 TA* out, int heads, int dv) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const int t = blockIdx.x;
  for (int idx = threadIdx.x; idx < heads * dv; idx += blockDim.x) {
    const float g = g_off >= 0 ? 1.f / (1.f + expf(-to_float(proj[(size_t)t * ldp + g_off + idx / dv]))) : 1.f;
    out[(size_t)t * heads * dv + idx] = from_float<TA>(to_float(in[(size_t)t * heads * dv + idx]) * g);
  }
}

// The same for bfloat16 rows whose heads are whole 16-byte pieces (dv a multiple of 8): a thread takes eight elements.
template <typename TP>
__global__ void head_gate_vec_kernel(const bf16* in, const TP* __restrict__ proj, long long ldp, int g_off, bf16* out,
                                     int heads, int dv, long long pieces) {
  pdl_wait();
  pdl_trigger();
  const int per_row = heads * dv / 8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < pieces;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / per_row;
    const int c = (int)(idx - t * per_row) * 8;
    const float g = 1.f / (1.f + expf(-to_float(proj[(size_t)t * ldp + g_off + c / dv])));
    uint4 v = *reinterpret_cast<const uint4*>(in + (size_t)t * heads * dv + c);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      h[i] = __floats2bfloat162_rn(f.x * g, f.y * g);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * heads * dv + c) = v;
  }
}

}  // namespace srlm

using namespace srlm;

#define SRLM_LATENT_TYPES(pd, wd, ...)                                                                     \
  do {                                                                                                     \
    if ((pd) == DT_F32 && (wd) == DT_F32) { using TP = float; using TW = float; __VA_ARGS__; }             \
    else if ((pd) == DT_F32 && (wd) == DT_BF16) { using TP = float; using TW = bf16; __VA_ARGS__; }        \
    else if ((pd) == DT_BF16 && (wd) == DT_BF16) { using TP = bf16; using TW = bf16; __VA_ARGS__; }        \
    else return refuse(ST_BAD_DTYPE, "latent attention: projection dtype %d with weight or cache dtype %d", \
                       (int)(pd), (int)(wd));                                                               \
  } while (0)

extern "C" int srlm_latent_append(const void* proj, int proj_dtype, long long ldp, int c_off, const float* norm_w,
                                  float eps, const float* cos_t, const float* sin_t, int pairs, int halves, void* cache,
                                  int cache_dtype, const int* kv_slot, int T, int rank, int rot, int q_col, int q_width,
                                  const float* q_norm_w, void* q_out, int q_dtype, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (rank <= 0 || rot < 0 || 2 * pairs > rot || c_off < 0 || ldp < c_off + rank + rot || !(eps > 0.f) ||
      (pairs > 0 && (!cos_t || !sin_t)) || (q_out && (q_width <= 0 || q_col < 0 || ldp < q_col + q_width || !q_norm_w)))
    return refuse(ST_BAD_SIZE, "latent_append: rank=%d rot=%d pairs=%d c_off=%d ldp=%lld", rank, rot, pairs, c_off, ldp);
#define SRLM_APPEND(TQ)                                                                                              \
  SRLM_LATENT_TYPES(proj_dtype, cache_dtype, (launch_pdl(latent_append_kernel<TP, TW, TQ>, dim3(T), dim3(128), 0, stream, \
      (const TP*)proj, ldp, c_off, norm_w, eps, cos_t, sin_t, pairs, halves, (TW*)cache, kv_slot, rank, rot, q_col,  \
      q_width, q_norm_w, (TQ*)q_out)))
  if (!q_out || q_dtype == DT_F32) SRLM_APPEND(float);
  else if (q_dtype == DT_BF16) SRLM_APPEND(bf16);
  else return refuse(ST_BAD_DTYPE, "latent_append: the normed queries' dtype %d", q_dtype);
#undef SRLM_APPEND
  return launched();
}

extern "C" int srlm_latent_absorb(const void* proj, int proj_dtype, long long ldp, const void* uk, int w_dtype,
                                  const float* cos_t, const float* sin_t, int pairs, int halves, float* q_out, int T, int heads,
                                  int dim, int rot, int rank, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const size_t smem = ((size_t)kTokTile * dim + (size_t)kProductWarps * kTokTile * kColTile) * sizeof(float);
  if (heads <= 0 || heads > 65535 || dim <= 0 || rank <= 0 || rot < 0 || 2 * pairs > rot || smem > 48 * 1024 ||
      ldp < (long long)heads * (dim + rot) || (pairs > 0 && (!cos_t || !sin_t)))
    return refuse(ST_BAD_SIZE, "latent_absorb: heads=%d dim=%d rot=%d rank=%d pairs=%d ldp=%lld", heads, dim, rot, rank,
                  pairs, ldp);
  dim3 grid((T + kTokTile - 1) / kTokTile, heads, (rank + kColTile - 1) / kColTile);
  SRLM_LATENT_TYPES(proj_dtype, w_dtype, (launch_pdl(latent_absorb_kernel<TP, TW>, dim3(grid), dim3(kProductWarps * 32), smem, stream, 
      (const TP*)proj, ldp, (const TW*)uk, cos_t, sin_t, pairs, halves, q_out, T, heads, dim, rot, rank)));
  return launched();
}

extern "C" int srlm_latent_expand(const float* o_lat, const void* uv_t, int w_dtype, const void* proj, int proj_dtype,
                                  long long ldp, int g_off, void* out, int out_dtype, int T, int heads, int rank,
                                  int dv, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const size_t smem = ((size_t)kTokTile * rank + (size_t)kProductWarps * kTokTile * kColTile) * sizeof(float);
  if (heads <= 0 || heads > 65535 || rank <= 0 || dv <= 0 || smem > 200 * 1024 || (g_off >= 0 && ldp < g_off + heads))
    return refuse(ST_BAD_SIZE, "latent_expand: heads=%d rank=%d dv=%d g_off=%d ldp=%lld", heads, rank, dv, g_off, ldp);
  dim3 grid((T + kTokTile - 1) / kTokTile, heads, (dv + kColTile - 1) / kColTile);
#define SRLM_EXPAND(TA)                                                                                          \
  do {                                                                                                           \
    auto kern = latent_expand_kernel<TP, TW, TA>;                                                                \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_pdl(kern, dim3(grid), dim3(kProductWarps * 32), smem, stream, o_lat, (const TW*)uv_t, (const TP*)proj, ldp, g_off, (TA*)out, T, heads,   \
                                      rank, dv);                                                                 \
  } while (0)
  if (out_dtype == DT_F32) SRLM_LATENT_TYPES(proj_dtype, w_dtype, SRLM_EXPAND(float));
  else if (out_dtype == DT_BF16) SRLM_LATENT_TYPES(proj_dtype, w_dtype, SRLM_EXPAND(bf16));
  else return refuse(ST_BAD_DTYPE, "latent_expand: output dtype %d", out_dtype);
#undef SRLM_EXPAND
  return launched();
}

extern "C" int srlm_latent_gather(const void* cache, int cache_dtype, void* dst, const int* block_table, int table_stride,
                                  const int* cu_kv, const int* kv_first, const int* kv_lens, int n_entries, int max_kv_len,
                                  int page_size, int width, int rank, cudaStream_t stream) {
  if (n_entries <= 0 || max_kv_len <= 0) return ST_OK;
  if (rank <= 0 || width < rank || page_size <= 0 || n_entries > 65535)
    return refuse(ST_BAD_SIZE, "latent_gather: rank=%d width=%d page_size=%d entries=%d", rank, width, page_size, n_entries);
  dim3 grid((unsigned)(max_kv_len < 4096 ? max_kv_len : 4096), (unsigned)n_entries);
  SRLM_DISPATCH_ACT(cache_dtype, TC, (launch_pdl(latent_gather_kernel<TC>, dim3(grid), dim3(64), 0, stream, 
      (const TC*)cache, (TC*)dst, block_table, table_stride, cu_kv, kv_first, kv_lens, page_size, width, rank)));
  return launched();
}

extern "C" int srlm_latent_rotate_q(const void* proj, int proj_dtype, long long ldp, const float* cos_t,
                                    const float* sin_t, int pairs, int halves, float* q_out, int T, int heads, int dim, int rot,
                                    cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (heads <= 0 || dim <= 0 || rot < 0 || 2 * pairs > rot || ldp < (long long)heads * (dim + rot) ||
      (pairs > 0 && (!cos_t || !sin_t)))
    return refuse(ST_BAD_SIZE, "latent_rotate_q: heads=%d dim=%d rot=%d pairs=%d ldp=%lld", heads, dim, rot, pairs, ldp);
  SRLM_DISPATCH_ACT(proj_dtype, TP, (launch_pdl(latent_rotate_q_kernel<TP>, dim3(T), dim3(256), 0, stream, 
      (const TP*)proj, ldp, cos_t, sin_t, pairs, halves, q_out, heads, dim, rot)));
  return launched();
}

// in: float32, or bfloat16 (then out may be the same buffer: an element is read and written by one thread)
extern "C" int srlm_head_gate(const void* in, int in_dtype, const void* proj, int proj_dtype, long long ldp, int g_off,
                              void* out, int out_dtype, int T, int heads, int dv, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (heads <= 0 || dv <= 0 || (g_off >= 0 && ldp < g_off + heads))
    return refuse(ST_BAD_SIZE, "head_gate: heads=%d dv=%d g_off=%d ldp=%lld", heads, dv, g_off, ldp);
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16 && g_off >= 0 && dv % 8 == 0 && ((((uintptr_t)in | (uintptr_t)out) & 15) == 0)) {
    const long long pieces = (long long)T * heads * dv / 8;
    const long long g = (pieces + 255) / 256;
    const dim3 grid((unsigned)(g > 148 * 16 ? 148 * 16 : g));
    if (proj_dtype == DT_F32)
      launch_pdl(head_gate_vec_kernel<float>, grid, dim3(256), 0, stream, (const bf16*)in, (const float*)proj, ldp, g_off, (bf16*)out, heads, dv, pieces);
    else
      launch_pdl(head_gate_vec_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)in, (const bf16*)proj, ldp, g_off, (bf16*)out, heads, dv, pieces);
    return launched();
  }
#define SRLM_GATE(TI, TP, TA) launch_pdl(head_gate_kernel<TI, TP, TA>, dim3(T), dim3(256), 0, stream, (const TI*)in, (const TP*)proj, ldp, g_off, (TA*)out, heads, dv)
  if (in_dtype == DT_F32 && proj_dtype == DT_F32 && out_dtype == DT_F32) SRLM_GATE(float, float, float);
  else if (in_dtype == DT_F32 && proj_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_GATE(float, float, bf16);
  else if (in_dtype == DT_F32 && proj_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_GATE(float, bf16, bf16);
  else if (in_dtype == DT_BF16 && proj_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_GATE(bf16, float, bf16);
  else if (in_dtype == DT_BF16 && proj_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_GATE(bf16, bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "head_gate: input dtype %d, projection dtype %d, output dtype %d", in_dtype, proj_dtype, out_dtype);
#undef SRLM_GATE
  return launched();
}
