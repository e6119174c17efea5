// A matrix memory with exponential gates: per head a state S [d, dv], a vector n [d] and a running maximum m of the
// gates' logarithms.  For every token, with i and f the logarithms of the input and forget gates,
//
//   m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k
//   o = S^T q / (max(|n . q|, exp(-m')) + floor)
//
// in float32, token by token.  The stacked projection row holds  q (H d) | k (H d) | v (H dv) | output gate (H dv) |
// i (H) | f (H), float32; i <- cap tanh((i + b_i) / cap), f <- log logistic(cap tanh((f + b_f) / cap)); q is scaled by
// 1 / sqrt(d).  A request's state row: S [H][dv][d] (a column of S, the d rows of one value element, is contiguous: a
// walking lane's rows are neighbours in memory) | n [H][d] | m [H], zeros for a new request.
//
// matrix_memory_recurrence: a block takes one entry, one head and a tile of the value columns; the tiles of a head are a
// thread-block cluster.  Its walking warps hold S: sixteen lanes share a column, a lane DPL neighbouring rows of it in
// registers, so S^T q is a sum in registers and four shuffles.  One more warp, the helper, runs a chunk of tokens
// ahead of them: it turns the chunk's gate logits into logarithms, walks m, forms exp(f + m - m') and exp(i - m') for
// every token, carries n (a lane holds d / 32 rows) and forms n . q and with it 1 / denominator; the walkers read these
// three numbers a token from shared memory and do nothing but S <- keep S + (write v) k and the read-out.  Every tile
// carries n this way; the first one writes it back.  All tiles read n and m before any of them writes: the cluster's
// barrier behind the loads orders that.  Tokens come in chunks of 16 through three buffers of shared memory (cp.async):
// while the walkers are on chunk c the helper is on chunk c + 1 and chunk c + 2 is in flight; one barrier a chunk.
// Rows of q and k lie in shared memory by lane, a few floats apart, so that the lanes' 16-byte loads meet no bank twice.
//
// matrix_memory_output: per token and head o / sqrt(mean(o^2) + eps) * w * logistic(gate), a warp a head.
#include "common.cuh"

namespace srlm {

constexpr int kMemChunk = 16;       // tokens of a chunk
constexpr int kMemLanes = 16;       // lanes of a column

__device__ __forceinline__ void mm_cp_async_4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void mm_cp_async_16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void mm_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int DPL>
__global__ void matrix_memory_recurrence_kernel(const float* __restrict__ proj, long long ldp, const float* __restrict__ bias_i,
                                                const float* __restrict__ bias_f, float cap, float floor_,
                                                float* __restrict__ state, long long state_stride,
                                                const int* __restrict__ cu_q, const int* __restrict__ slots,
                                                float* __restrict__ o_out, int H, int d, int dv, int cols, int vec, int nbuf) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float mm_smem[];
  constexpr int LS = DPL == 4 ? 4 : DPL + 4;       // a lane's rows, padded (8 lanes' 16-byte loads then meet 8 groups of banks)
  constexpr int QS = kMemLanes * LS;               // a token's q (or k) row in shared memory
  constexpr int DN = (kMemLanes * DPL + 31) / 32;  // rows of n a helper lane holds
  // raw chunks, three buffers of: q [chunk][QS] | k [chunk][QS] | v [chunk][cols] | gate logits [chunk][2];
  // then two buffers of what the helper makes of a chunk: keep | write | 1 / denominator [chunk] each; then its scratch
  const int per_raw = kMemChunk * (2 * QS + cols + 2);
  float* coef = mm_smem + nbuf * per_raw;           // nbuf: 3, or 1 when no entry of the step has more than one chunk
  float* part = coef + 2 * 3 * kMemChunk;          // [chunk][33]: the helper lanes' shares of n . q
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * cols;
  const int first = cu_q[e], n_tok = cu_q[e + 1] - first;
  const int walkers = cols * kMemLanes;            // threads that hold S; the last warp of the block is the helper
  const bool helper = (int)threadIdx.x >= walkers;
  const int lane = threadIdx.x & 31;
  const int col_local = threadIdx.x / kMemLanes, l = threadIdx.x % kMemLanes;
  const int col = c0 + col_local;
  const bool live = !helper && col < dv;
  float* row = state + (size_t)slots[e] * state_stride;
  float* S_g = row + (size_t)h * d * dv;
  float* n_g = row + (size_t)H * d * dv + (size_t)h * d;
  float* m_g = row + (size_t)H * d * dv + (size_t)H * d + h;
  const int q_off = h * d, k_off = H * d + h * d, v_off = 2 * H * d + h * dv + c0, i_off = 2 * H * d + 2 * H * dv + h,
            f_off = i_off + H;
  const int chunks = (n_tok + kMemChunk - 1) / kMemChunk;
  const int rows_pad = kMemLanes * DPL;

  auto fetch = [&](int chunk) {
    if (chunk < chunks) {
      float* base = mm_smem + (chunk % nbuf) * per_raw;
      const int t0 = chunk * kMemChunk, cnt = min(kMemChunk, n_tok - t0);
      if (vec) {        // 16-byte copies: four neighbouring rows of q and of k, four neighbouring columns of v
        constexpr int RP4 = kMemLanes * DPL / 4;
        for (int idx = threadIdx.x; idx < cnt * RP4; idx += blockDim.x) {
          const int tt = idx / RP4, r = (idx - tt * RP4) * 4;
          const int at = tt * QS + (r / DPL) * LS + r % DPL;
          if (r < d) {
            const float* src = proj + (size_t)(first + t0 + tt) * ldp;
            mm_cp_async_16(base + at, src + q_off + r);
            mm_cp_async_16(base + kMemChunk * QS + at, src + k_off + r);
          } else {
            *reinterpret_cast<float4*>(base + at) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(base + kMemChunk * QS + at) = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        const int c4 = cols / 4;
        for (int idx = threadIdx.x; idx < cnt * c4; idx += blockDim.x) {
          const int tt = idx / c4, c = (idx - tt * c4) * 4;
          if (c0 + c < dv) mm_cp_async_16(base + 2 * kMemChunk * QS + tt * cols + c, proj + (size_t)(first + t0 + tt) * ldp + v_off + c);
        }
      } else {
        for (int idx = threadIdx.x; idx < cnt * rows_pad; idx += blockDim.x) {
          const int tt = idx / rows_pad, r = idx - tt * rows_pad;
          const int at = tt * QS + (r / DPL) * LS + r % DPL;
          if (r < d) {
            const float* src = proj + (size_t)(first + t0 + tt) * ldp;
            mm_cp_async_4(base + at, src + q_off + r);
            mm_cp_async_4(base + kMemChunk * QS + at, src + k_off + r);
          } else {
            base[at] = 0.f;
            base[kMemChunk * QS + at] = 0.f;
          }
        }
        for (int idx = threadIdx.x; idx < cnt * cols; idx += blockDim.x) {
          const int tt = idx / cols, c = idx - tt * cols;
          if (c0 + c < dv) mm_cp_async_4(base + 2 * kMemChunk * QS + tt * cols + c, proj + (size_t)(first + t0 + tt) * ldp + v_off + c);
        }
      }
      for (int idx = threadIdx.x; idx < cnt * 2; idx += blockDim.x)
        mm_cp_async_4(base + kMemChunk * (2 * QS + cols) + idx,
                      proj + (size_t)(first + t0 + (idx >> 1)) * ldp + ((idx & 1) ? f_off : i_off));
    }
    asm volatile("cp.async.commit_group;" ::);
  };

  // the helper's state: n (rows lane * DN + j) and m; the walkers': DPL rows of a column of S
  float S[DPL], nv[DN];
  float m = 0.f;
  if (helper) {
#pragma unroll
    for (int j = 0; j < DN; ++j) {
      const int r = lane * DN + j;
      nv[j] = r < d ? n_g[r] : 0.f;
    }
    m = *m_g;
  } else {
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int r = l * DPL + j;
      S[j] = (live && r < d) ? S_g[(size_t)col * d + r] : 0.f;
    }
  }
  fetch(0);
  fetch(1);
  mm_cluster_sync();                 // every tile of this head holds the old n and m before any tile writes new ones
  const float q_scale = rsqrtf((float)d);

  // what the helper makes of chunk ch (its raw data has landed and is visible): keep, write, 1 / denominator per token
  auto prepare = [&](int ch) {
    float* base = mm_smem + (ch % nbuf) * per_raw;
    const float* q_s = base;
    const float* k_s = base + kMemChunk * QS;
    float* g_s = base + kMemChunk * (2 * QS + cols);
    float* cf = coef + (ch & 1) * 3 * kMemChunk;
    const int cnt = min(kMemChunk, n_tok - ch * kMemChunk);
    // the gates' logarithms, a lane a token, in place
    float gi = 0.f, gf = 0.f;
    if (lane < cnt) {
      gi = cap * tanhf((g_s[2 * lane] + bias_i[h]) / cap);
      const float z = cap * tanhf((g_s[2 * lane + 1] + bias_f[h]) / cap);
      gf = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));           // log logistic(z)
      g_s[2 * lane] = gi;
      g_s[2 * lane + 1] = gf;
    }
    __syncwarp();
    // m walks the chunk in every lane's registers; lane t keeps token t's
    float m_mine = 0.f, m_before = 0.f;
#pragma unroll
    for (int tt = 0; tt < kMemChunk; ++tt) {
      if (tt < cnt) {
        const float m_new = fmaxf(g_s[2 * tt + 1] + m, g_s[2 * tt]);
        if (lane == tt) { m_before = m; m_mine = m_new; }
        m = m_new;
      }
    }
    if (lane < cnt) {
      cf[lane] = expf(gf + m_before - m_mine);
      cf[kMemChunk + lane] = expf(gi - m_mine);
    }
    __syncwarp();
    // n walks the chunk; a lane's share of n . q of every token goes through shared memory to the token's lane.  A lane's
    // DN rows are neighbours within one walker lane's rows.
    const int off = ((lane * DN) / DPL) * LS + (lane * DN) % DPL;
#pragma unroll
    for (int tt = 0; tt < kMemChunk; ++tt) {
      if (tt < cnt) {
        const float kp = cf[tt], wr = cf[kMemChunk + tt];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < DN; ++j) {
          const float kk = k_s[tt * QS + off + j], qq = q_s[tt * QS + off + j];
          nv[j] = fmaf(kp, nv[j], wr * kk);
          acc = fmaf(nv[j], qq, acc);
        }
        part[tt * 33 + lane] = acc;
      }
    }
    __syncwarp();
    if (lane < cnt) {
      float nq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        nq[0] += part[lane * 33 + i];
        nq[1] += part[lane * 33 + i + 1];
        nq[2] += part[lane * 33 + i + 2];
        nq[3] += part[lane * 33 + i + 3];
      }
      const float total = (nq[0] + nq[1]) + (nq[2] + nq[3]);
      cf[2 * kMemChunk + lane] = q_scale / (fmaxf(fabsf(total * q_scale), expf(-m_mine)) + floor_);
    }
    __syncwarp();
  };

  asm volatile("cp.async.wait_group 1;" ::);       // chunk 0 has landed
  __syncthreads();
  if (helper) prepare(0);
  for (int ch = 0; ch < chunks; ++ch) {
    asm volatile("cp.async.wait_group 0;" ::);     // chunk ch + 1 has landed (this thread's copies)
    __syncthreads();                               // ... and everybody's; the helper's work on chunk ch is visible; nobody
    fetch(ch + 2);                                 // reads chunk ch - 1 any more, whose buffer chunk ch + 2 takes
    if (helper) {
      if (ch + 1 < chunks) prepare(ch + 1);
    } else {
      const float* base = mm_smem + (ch % nbuf) * per_raw;
      const float* q_s = base + l * LS;
      const float* k_s = base + kMemChunk * QS + l * LS;
      const float* v_s = base + 2 * kMemChunk * QS;
      const float* cf = coef + (ch & 1) * 3 * kMemChunk;
      const int cnt = min(kMemChunk, n_tok - ch * kMemChunk);
      float* o_row = o_out + (size_t)(first + ch * kMemChunk) * H * dv + (size_t)h * dv + col;
      // a lane's share of S^T q for every token of the chunk; the shares cross the sixteen lanes once a chunk
      float share[kMemChunk];
#pragma unroll
      for (int tt = 0; tt < kMemChunk; ++tt) {
        share[tt] = 0.f;
        if (tt < cnt) {
          const float keep = cf[tt];
          const float wv = cf[kMemChunk + tt] * v_s[tt * cols + col_local];      // (a column beyond dv: rubbish that is never written)
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int j = 0; j < DPL; j += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(k_s + tt * QS + j);
            const float4 qq = *reinterpret_cast<const float4*>(q_s + tt * QS + j);
            S[j] = fmaf(keep, S[j], wv * kk.x);
            S[j + 1] = fmaf(keep, S[j + 1], wv * kk.y);
            S[j + 2] = fmaf(keep, S[j + 2], wv * kk.z);
            S[j + 3] = fmaf(keep, S[j + 3], wv * kk.w);
            acc[0] = fmaf(S[j], qq.x, acc[0]);
            acc[1] = fmaf(S[j + 1], qq.y, acc[1]);
            acc[2] = fmaf(S[j + 2], qq.z, acc[2]);
            acc[3] = fmaf(S[j + 3], qq.w, acc[3]);
          }
          share[tt] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
      }
      // halving exchanges: after the step with distance w a lane holds w sums, those of the tokens that share its bits
      // above w; in the end lane l holds token l's
#pragma unroll
      for (int w = kMemChunk / 2; w >= 1; w >>= 1) {
        const bool upper = (l & w) != 0;
#pragma unroll
        for (int i = 0; i < w; ++i) {
          const float send = upper ? share[i] : share[i + w];
          const float mine = upper ? share[i + w] : share[i];
          share[i] = mine + __shfl_xor_sync(0xffffffffu, send, w);
        }
      }
      if (live && l < cnt) o_row[(size_t)l * H * dv] = share[0] * cf[2 * kMemChunk + l];
    }
  }
  if (helper) {
    if (blockIdx.x == 0) {
#pragma unroll
      for (int j = 0; j < DN; ++j) {
        const int r = lane * DN + j;
        if (r < d) n_g[r] = nv[j];
      }
      if (lane == 0) *m_g = m;
    }
  } else if (live) {
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const int r = l * DPL + j;
      if (r < d) S_g[(size_t)col * d + r] = S[j];
    }
  }
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
                                             const int* cu_q, const int* slots, float* o_out, int n_entries, int max_q_len,
                                             int H, int d, int dv, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (H <= 0 || d <= 0 || dv <= 0 || d > 256 || !(cap > 0.f) || ldp < 2LL * H * d + 2LL * H * dv + 2 * H ||
      state_stride < (long long)H * d * dv + (long long)H * d + H || n_entries > 65535 || H > 65535)
    return refuse(ST_BAD_SIZE, "matrix_memory_recurrence: heads=%d dim=%d (at most 256) vdim=%d ld=%lld", H, d, dv, ldp);
  // the value columns of a head in up to 8 tiles (a cluster), each of a multiple of 4 columns (whole warps)
  int tiles = (dv + 15) / 16;
  if (tiles > 8) tiles = 8;
  int cols = ((dv + tiles - 1) / tiles + 3) / 4 * 4;
  tiles = (dv + cols - 1) / cols;
  const int threads = cols * kMemLanes + 32;      // the walkers and the helper warp
  if (threads > 1024) return refuse(ST_BAD_SIZE, "matrix_memory_recurrence: vdim=%d (at most 480)", dv);
  const int dpl_rows = (d + kMemLanes - 1) / kMemLanes;
  const int dpl_t = dpl_rows <= 4 ? 4 : dpl_rows <= 8 ? 8 : 16;
  const int ls = dpl_t == 4 ? 4 : dpl_t + 4;
  // steps whose entries all fit one chunk (decode steps) need one buffer of raw tokens, and more blocks fit an SM
  const int nbuf = max_q_len > 0 && max_q_len <= kMemChunk ? 1 : 3;
  const size_t smem = ((size_t)nbuf * kMemChunk * (2 * kMemLanes * ls + cols + 2) + 2 * 3 * kMemChunk + kMemChunk * 33) * sizeof(float);
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
  const int dpl = dpl_t;
  const int vec = ldp % 4 == 0 && d % 4 == 0 && dv % 4 == 0 && ((uintptr_t)proj & 15) == 0;     // 16-byte copies into the chunks
#define SRLM_MM(DPL)                                                                                                     \
  do {                                                                                                                   \
    auto kern = matrix_memory_recurrence_kernel<DPL>;                                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    cudaLaunchKernelEx(&cfg, kern, proj, ldp, bias_i, bias_f, cap, floor_, state, state_stride, cu_q, slots, o_out, H, d, \
                       dv, cols, vec, nbuf);                                                                             \
  } while (0)
  if (dpl <= 4) SRLM_MM(4);
  else if (dpl <= 8) SRLM_MM(8);
  else SRLM_MM(16);
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
