// A matrix memory with exponential gates: per head a state S [d, dv], a vector n [d] and a running maximum m of the
// gates' logarithms.  For every token, with i and f the logarithms of the input and forget gates,
//
//   m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k
//   o = S^T q / (max(|n . q|, exp(-m')) + floor)
//
// in float32, token by token.  The stacked projection row holds  q (H d) | k (H d) | v (H dv) | output gate (H dv) |
// i (H) | f (H), float32; i <- cap tanh((i + b_i) / cap), f <- log logistic(cap tanh((f + b_f) / cap)); q is scaled by
// 1 / sqrt(d).  A request's state row: S [H][d][dv] | n [H][d] | m [H], zeros for a new request.
//
// matrix_memory_recurrence: a block takes one entry, one head and a tile of the value columns; the tiles of a head are a
// thread-block cluster.  Eight lanes share a column of S (a lane holds the rows r = lane + 8 j in registers), so S^T q is
// a sum in registers and three shuffles.  Every tile also carries n (it needs n . q); the first one writes it back.  All
// tiles read n and m before any of them writes: the cluster's barrier behind the loads orders that.  Tokens come in
// chunks through shared memory (cp.async, the next chunk in flight while this one is walked); the gates' transforms are
// applied once per chunk.
//
// matrix_memory_output: per token and head o / sqrt(mean(o^2) + eps) * w * logistic(gate), a warp a head.
#include "common.cuh"

namespace srlm {

constexpr int kMemChunk = 16;       // tokens of a chunk
constexpr int kMemLanes = 8;        // lanes of a column

__device__ __forceinline__ void mm_cp_async_4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void mm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int DPL>
__global__ void matrix_memory_recurrence_kernel(const float* __restrict__ proj, long long ldp, const float* __restrict__ bias_i,
                                                const float* __restrict__ bias_f, float cap, float floor_,
                                                float* __restrict__ state, long long state_stride,
                                                const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                float* __restrict__ o_out, int H, int d, int dv, int cols) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float mm_smem[];
  // two buffers of: q [chunk][d] | k [chunk][d] | v [chunk][cols] | gates [chunk][2]
  const int per_buf = kMemChunk * (2 * d + cols + 2);
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cols;
  const int first = cu_q[e], n_tok = cu_q[e + 1] - first;
  const int col_local = threadIdx.x / kMemLanes, l = threadIdx.x % kMemLanes;
  const int col = c0 + col_local;
  const bool live = col_local < cols && col < dv;
  float* row = state + (size_t)slots[e] * state_stride;
  float* S_g = row + (size_t)h * d * dv;
  float* n_g = row + (size_t)H * d * dv + (size_t)h * d;
  float* m_g = row + (size_t)H * d * dv + (size_t)H * d + h;
  const int q_off = h * d, k_off = H * d + h * d, v_off = 2 * H * d + h * dv + c0, i_off = 2 * H * d + 2 * H * dv + h,
            f_off = i_off + H;

  auto fetch = [&](int chunk, int buf) {
    float* base = mm_smem + buf * per_buf;
    const int t0 = chunk * kMemChunk, cnt = min(kMemChunk, n_tok - t0);
    for (int idx = threadIdx.x; idx < cnt * d; idx += blockDim.x) {
      const int tt = idx / d, r = idx - tt * d;
      const float* src = proj + (size_t)(first + t0 + tt) * ldp;
      mm_cp_async_4(base + tt * d + r, src + q_off + r);
      mm_cp_async_4(base + kMemChunk * d + tt * d + r, src + k_off + r);
    }
    for (int idx = threadIdx.x; idx < cnt * cols; idx += blockDim.x) {
      const int tt = idx / cols, c = idx - tt * cols;
      if (c0 + c < dv) mm_cp_async_4(base + 2 * kMemChunk * d + tt * cols + c, proj + (size_t)(first + t0 + tt) * ldp + v_off + c);
    }
    for (int idx = threadIdx.x; idx < cnt * 2; idx += blockDim.x) {
      const int tt = idx >> 1, which = idx & 1;
      mm_cp_async_4(base + kMemChunk * (2 * d + cols) + idx, proj + (size_t)(first + t0 + tt) * ldp + (which ? f_off : i_off));
    }
    asm volatile("cp.async.commit_group;" ::);
  };

  float S[DPL], nv[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int r = l + kMemLanes * j;
    S[j] = (live && r < d) ? S_g[(size_t)r * dv + col] : 0.f;
    nv[j] = r < d ? n_g[r] : 0.f;
  }
  float m = *m_g;
  const int chunks = (n_tok + kMemChunk - 1) / kMemChunk;
  fetch(0, 0);
  mm_cluster_sync();                 // every tile of this head holds the old n and m before any tile writes new ones
  const float q_scale = rsqrtf((float)d);
  for (int ch = 0; ch < chunks; ++ch) {
    const int buf = ch & 1;
    if (ch + 1 < chunks) {
      fetch(ch + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::);
    } else {
      asm volatile("cp.async.wait_group 0;" ::);
    }
    __syncthreads();
    float* base = mm_smem + buf * per_buf;
    const float* q_s = base;
    const float* k_s = base + kMemChunk * d;
    const float* v_s = base + 2 * kMemChunk * d;
    float* g_s = base + kMemChunk * (2 * d + cols);
    const int cnt = min(kMemChunk, n_tok - ch * kMemChunk);
    if (threadIdx.x < 2 * cnt) {       // the gates' logarithms, once per token
      const int which = threadIdx.x & 1;
      const float z = cap * tanhf((g_s[threadIdx.x] + (which ? bias_f[h] : bias_i[h])) / cap);
      // log logistic(z) = min(z, 0) - log1p(exp(-|z|))
      g_s[threadIdx.x] = which ? fminf(z, 0.f) - log1pf(expf(-fabsf(z))) : z;
    }
    __syncthreads();
    for (int tt = 0; tt < cnt; ++tt) {
      const float gi = g_s[2 * tt], gf = g_s[2 * tt + 1];
      const float m_new = fmaxf(gf + m, gi);
      const float keep = expf(gf + m - m_new), write = expf(gi - m_new);
      m = m_new;
      const float wv = live ? write * v_s[tt * cols + col_local] : 0.f;
      float acc_o = 0.f, acc_n = 0.f;
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        const int r = l + kMemLanes * j;
        const float kk = r < d ? k_s[tt * d + r] : 0.f, qq = r < d ? q_s[tt * d + r] : 0.f;
        S[j] = fmaf(keep, S[j], wv * kk);
        nv[j] = fmaf(keep, nv[j], write * kk);
        acc_o = fmaf(S[j], qq, acc_o);
        acc_n = fmaf(nv[j], qq, acc_n);
      }
#pragma unroll
      for (int o = 1; o < kMemLanes; o <<= 1) {
        acc_o += __shfl_xor_sync(0xffffffffu, acc_o, o);
        acc_n += __shfl_xor_sync(0xffffffffu, acc_n, o);
      }
      if (l == 0 && live) {
        const float den = fmaxf(fabsf(acc_n * q_scale), expf(-m)) + floor_;
        o_out[(size_t)(first + ch * kMemChunk + tt) * H * dv + (size_t)h * dv + col] = acc_o * q_scale / den;
      }
    }
    __syncthreads();                   // the buffer is free for the chunk after the next
  }
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    const int r = l + kMemLanes * j;
    if (live && r < d) S_g[(size_t)r * dv + col] = S[j];
    if (blockIdx.x == 0 && col_local == 0 && r < d) n_g[r] = nv[j];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *m_g = m;
}

template <typename TO>
__global__ void matrix_memory_output_kernel(const float* __restrict__ o, const float* __restrict__ norm_w, float eps,
                                            const float* __restrict__ proj, long long ldp, int g_off, TO* __restrict__ out,
                                            long long heads_total, int H, int dv) {
  pdl_wait();
  pdl_trigger();
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= heads_total) return;
  const int lane = threadIdx.x & 31;
  const long long t = warp / H;
  const int h = (int)(warp % H);
  const float* src = o + (size_t)t * H * dv + (size_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += src[i] * src[i];
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float g = 1.f / (1.f + expf(-proj[(size_t)t * ldp + g_off + h * dv + i]));
    out[(size_t)t * H * dv + (size_t)h * dv + i] = from_float<TO>(src[i] * inv * norm_w[h * dv + i] * g);
  }
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_matrix_memory_state_size(int H, int d, int dv) { return H * d * dv + H * d + H; }

// proj float32 [T, ldp] as laid out above; state float32 [slots, state_stride]; o_out float32 [T, H dv]
extern "C" int srlm_matrix_memory_recurrence(const float* proj, long long ldp, const float* bias_i, const float* bias_f,
                                             float cap, float floor_, float* state, long long state_stride,
                                             const int* cu_q, const int* slots, float* o_out, int n_entries, int H, int d,
                                             int dv, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (H <= 0 || d <= 0 || dv <= 0 || d > 256 || !(cap > 0.f) || ldp < 2LL * H * d + 2LL * H * dv + 2 * H ||
      state_stride < (long long)H * d * dv + (long long)H * d + H || n_entries > 65535 || H > 65535)
    return refuse(ST_BAD_SIZE, "matrix_memory_recurrence: heads=%d dim=%d (at most 256) vdim=%d ld=%lld", H, d, dv, ldp);
  // the value columns of a head in up to 8 tiles (a cluster), each of a multiple of 4 columns (whole warps)
  int tiles = (dv + 15) / 16;
  if (tiles > 8) tiles = 8;
  int cols = ((dv + tiles - 1) / tiles + 3) / 4 * 4;
  tiles = (dv + cols - 1) / cols;
  const int threads = cols * kMemLanes;
  if (threads > 1024) return refuse(ST_BAD_SIZE, "matrix_memory_recurrence: vdim=%d (at most 1024)", dv);
  const size_t smem = 2 * (size_t)kMemChunk * (2 * d + cols + 2) * sizeof(float);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)tiles, (unsigned)H, (unsigned)n_entries);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)tiles;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int dpl = (d + kMemLanes - 1) / kMemLanes;
#define SRLM_MM(DPL)                                                                                                     \
  do {                                                                                                                   \
    auto kern = matrix_memory_recurrence_kernel<DPL>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    cudaLaunchKernelEx(&cfg, kern, proj, ldp, bias_i, bias_f, cap, floor_, state, state_stride, cu_q, slots, o_out, H, d, \
                       dv, cols);                                                                                        \
  } while (0)
  if (dpl <= 4) SRLM_MM(4);
  else if (dpl <= 8) SRLM_MM(8);
  else if (dpl <= 16) SRLM_MM(16);
  else SRLM_MM(32);
#undef SRLM_MM
  return launched();
}

// o float32 [T, H dv]; norm_w float32 [H dv]; the gate's logits: columns g_off .. of proj; out [T, H dv]
extern "C" int srlm_matrix_memory_output(const float* o, const float* norm_w, float eps, const float* proj, long long ldp,
                                         int g_off, void* out, int out_dtype, int T, int H, int dv, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (H <= 0 || dv <= 0 || !(eps > 0.f) || g_off < 0 || ldp < g_off + (long long)H * dv)
    return refuse(ST_BAD_SIZE, "matrix_memory_output: heads=%d vdim=%d g_off=%d ld=%lld", H, dv, g_off, ldp);
  const long long total = (long long)T * H;
  SRLM_DISPATCH_ACT(out_dtype, TO, launch_pdl(matrix_memory_output_kernel<TO>, dim3((unsigned)((total + 3) / 4)), dim3(128),
                                              0, stream, o, norm_w, eps, proj, ldp, g_off, (TO*)out, total, H, dv));
  return launched();
}
