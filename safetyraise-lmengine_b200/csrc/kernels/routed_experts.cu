// A feed-forward of routed experts: every token runs the `top` experts with the largest router logits and
// adds their outputs, weighted by the softmax over those logits alone (scoring 0), or by the logistic of each
// chosen logit, not renormalised (scoring 1), or by the softmax over ALL experts' logits, renormalised over the chosen
// ones (scoring 2; the experts may then form equal groups of neighbours of which only the best few, judged by their
// largest score, can be chosen).  A weight multiplies its expert's output (in `combine`) or, for
// experts without biases, its input: then the first grouped product scales its gate and up sums by the pair's
// weight before the activation (W (w h) = w (W h)), and `combine` adds the rows as they are.
//
//   route    router logits (+ bias) -> the chosen experts and their weights, per token (float32)
//   sort     the (token, choice) pairs ordered by expert: where each expert's rows start, which pair
//            sits in which row, and how many tiles of kTile rows each expert has
//   grouped  C[row] = A[row's token] . W[row's expert]^T for all experts in one launch; with the gated
//            activation in its epilogue for the experts' first product
//   combine  out[token] = sum over its choices, in the order of the choices, of weight * row (+ the
//            output of the expert that every token runs)
//
// Nothing here depends on what else is in the batch: a row's sums run over k in index order whatever
// tile the row landed in, and the combination adds a token's rows in the order of its choices.
// Everything is sized on the host by upper bounds (pairs / kTile + experts tiles), so a step's launches
// depend on its token count alone and can be replayed from a CUDA graph.
//
// The gated activation of an expert: with limit > 0 the "clamped GLU", g = min(gate, limit), u = clamp(up, -limit,
// limit), y = g * logistic(alpha * g) * (u + 1); with limit <= 0 the plain one, y = gate * logistic(gate) * up.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int kTile = 64;        // rows (token, choice pairs) of a tile of the grouped products

__device__ __forceinline__ float clamped_glu(float gate, float up, float limit, float alpha) {
  if (!(limit > 0.f)) return gate * (1.f / (1.f + expf(-gate))) * up;
  const float g = fminf(gate, limit);
  const float u = fminf(fmaxf(up, -limit), limit);
  return g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f);
}

// The activation of an expert without a gate: 0 none, 1 the exact gelu.
__device__ __forceinline__ float plain_activation(float z, int act) {
  return act == 1 ? 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)) : z;
}

// One warp routes a token.  The row of logits sits in shared memory (z: E floats of the warp's own); `top` times
// the warp takes the largest value left (ties: the lowest index) and strikes it out.  weights = softmax over the
// chosen values; scoring 1: weight = logistic of the chosen value itself.
__device__ __forceinline__ void route_token(const float* __restrict__ logits, long long ld, const float* __restrict__ bias,
                                            int t, int E, int top, float* z, int* __restrict__ choice,
                                            float* __restrict__ weight, int scoring, int groups, int kept) {
  const int lane = threadIdx.x & 31;
  for (int e = lane; e < E; e += 32) z[e] = logits[(size_t)t * ld + e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  float first = 0.f, sum = 0.f;
  float z_max = 0.f, z_den = 1.f;          // scoring 2: score(e) = exp(z[e] - z_max) / z_den
  if (scoring == 2) {
    float mx = -CUDART_INF_F;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    z_max = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) den += expf(z[e] - z_max);
    z_den = warp_sum(den);
    if (groups > 1 && kept < groups) {
      // a group counts as its largest logit (the softmax keeps the order); `kept` times the best group left is marked
      // (ties: the lowest index); the experts of unmarked groups are struck out.  Lane l owns groups l, l + 32, ...
      const int per = E / groups;
      uint32_t mine = 0;
      for (int c = 0; c < kept; ++c) {
        float best = -CUDART_INF_F;
        int at = groups;
        for (int g = lane, i = 0; g < groups; g += 32, ++i) {
          if ((mine >> i) & 1u) continue;
          float gm = -CUDART_INF_F;
          for (int e = g * per; e < (g + 1) * per; ++e) gm = fmaxf(gm, z[e]);
          if (gm > best || (gm == best && g < at)) { best = gm; at = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, at, o);
          if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at < groups && (at & 31) == lane) mine |= 1u << (at >> 5);
      }
      for (int g = lane, i = 0; g < groups; g += 32, ++i)
        if (!((mine >> i) & 1u))
          for (int e = g * per; e < (g + 1) * per; ++e) z[e] = -CUDART_INF_F;
      __syncwarp();
    }
  }
  for (int c = 0; c < top; ++c) {
    float best = -CUDART_INF_F;
    int at = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }     // NaN never wins: a struck-out slot is -inf
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at >= E) at = c < E ? c : 0;            // a row of NaN: any valid expert; the step's finite check reports it
    if (c == 0) first = best;
    const float p = scoring == 1 ? 1.f / (1.f + expf(-best)) : scoring == 2 ? expf(best - z_max) / z_den : expf(best - first);
    sum += p;
    if (lane == 0) {
      choice[(size_t)t * top + c] = at;
      weight[(size_t)t * top + c] = p;
      z[at] = -CUDART_INF_F;
    }
    __syncwarp();
  }
  __syncwarp();
  if (scoring == 0)
    for (int c = lane; c < top; c += 32) weight[(size_t)t * top + c] /= sum;
  if (scoring == 2)
    for (int c = lane; c < top; c += 32) weight[(size_t)t * top + c] /= sum + 1e-20f;
  __syncwarp();
}

__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias,
                                 int T, int E, int top, int* __restrict__ choice, float* __restrict__ weight, int scoring,
                                 int groups, int kept) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float route_smem[];
  const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + warp;
  if (t >= T) return;
  route_token(logits, ld, bias, t, E, top, route_smem + (size_t)warp * E, choice, weight, scoring, groups, kept);
}

// One block.  offsets[E + 1]: first row of each expert; tiles[E + 1]: first tile of each expert (tiles of
// tile_rows rows, none shared by two experts); pair_of_row[n]; row_of_pair[n].  Which row of its expert a pair
// gets depends on the order the threads arrive in; no result depends on it.
// align: every expert's rows start at a multiple of tile_rows (for products whose tiles are fixed rows of their
// operands); pair_of_row then has rows_cap entries, -1 where a row holds no pair, and group_of_tile[max_tiles]
// names the expert of every tile, -1 for a tile without rows.
// logits != null: the block first routes the n / top tokens itself (small steps: one launch fewer), a warp a
// token at a time, and writes choice and weight; then it orders what it chose.
__global__ void moe_sort_kernel(int* __restrict__ choice, int n, int E, int tile_rows, int align,
                                int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ pair_of_row,
                                int* __restrict__ row_of_pair, int* __restrict__ group_of_tile, int max_tiles, int rows_cap,
                                const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int top,
                                float* __restrict__ weight, int scoring, int groups, int kept) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int sort_smem[];
  int* count = sort_smem;            // [E]
  int* start = count + E;            // [E + 1]
  if (logits) {
    float* z = reinterpret_cast<float*>(start + E + 1) + (size_t)(threadIdx.x >> 5) * E;
    for (int t = threadIdx.x >> 5; t < n / top; t += blockDim.x >> 5) route_token(logits, ld, bias, t, E, top, z, choice, weight, scoring, groups, kept);
    __syncthreads();                 // the choices of all tokens are written (and visible to the block)
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  if (align) {
    for (int i = threadIdx.x; i < rows_cap; i += blockDim.x) pair_of_row[i] = -1;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) group_of_tile[i] = -1;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = choice[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tl = 0;
    for (int e = 0; e < E; ++e) {
      if (align) rows = tl * tile_rows;
      start[e] = rows;
      offsets[e] = rows;
      tiles[e] = tl;
      rows += count[e];
      const int nt = (count[e] + tile_rows - 1) / tile_rows;
      if (align)
        for (int i = tl; i < tl + nt && i < max_tiles; ++i) group_of_tile[i] = e;
      tl += nt;
    }
    start[E] = rows;
    offsets[E] = rows;
    tiles[E] = tl;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;       // now the cursor of each expert
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = choice[i];
    if (e < 0 || e >= E) { row_of_pair[i] = -1; continue; }
    const int row = start[e] + atomicAdd(&count[e], 1);
    pair_of_row[row] = i;
    row_of_pair[i] = row;
  }
}

// xs[row, :] = x[pair_of_row[row] / pairs_per_token, :], zeros for a row without a pair; 16 bytes a thread.
// pair_scale (float32 [pairs] or null): the row is multiplied by its pair's number (a weight on an expert's input).
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ pair_of_row,
                                       int pairs_per_token, bf16* __restrict__ xs, int rows, int K,
                                       const float* __restrict__ pair_scale) {
  pdl_wait();
  pdl_trigger();
  const int vecs = K / 8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)rows * vecs;
       idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx / vecs), c = (int)(idx - (long long)row * vecs);
    const int pair = pair_of_row[row];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pair >= 0) v = *reinterpret_cast<const uint4*>(x + (size_t)(pair / pairs_per_token) * ldx + c * 8);
    if (pair >= 0 && pair_scale) {
      const float w = pair_scale[pair];
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        h2[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
    }
    *reinterpret_cast<uint4*>(xs + (size_t)row * K + c * 8) = v;
  }
}

// The expert and the first row of tile `tile`; false when the step has fewer tiles.
__device__ __forceinline__ bool tile_home(const int* __restrict__ offsets, const int* __restrict__ tiles, int E, int tile,
                                          int& expert, int& row0, int& row_end) {
  if (tile >= tiles[E]) return false;
  int lo = 0, hi = E - 1;                                   // the last expert whose first tile is <= tile
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tiles[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  expert = lo;
  row0 = offsets[lo] + (tile - tiles[lo]) * kTile;
  row_end = offsets[lo + 1];
  return true;
}

// Float32 arithmetic (FMA), any sizes: the float32 path, and sizes the tensor-core form does not take.
// GLU: W holds per expert the gate rows of all features, then the up rows (interleaved == 0), or blocks
// of 16 rows, 8 gate rows then the 8 up rows of the same features (interleaved == 1); C gets the
// activation, N features wide.  Else C[row, 0..N) = A . W[expert]^T, N weight rows per expert.
constexpr int GBN = 64, GBK = 16;

template <typename TA, typename TW, typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_grouped_simt_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ pair_of_row, int pairs_per_token,
                        const TW* __restrict__ W, TO* __restrict__ C, long long ldc, const int* __restrict__ offsets,
                        const int* __restrict__ tiles, int E, int N, int K, int interleaved, float limit, float alpha,
                        const float* __restrict__ pair_scale, int act) {
  pdl_wait();
  pdl_trigger();
  __shared__ float As[GBK][kTile + 4];
  __shared__ float Ws[GBK][GBN + 4];
  __shared__ float Us[GLU ? GBK : 1][GBN + 4];
  __shared__ int a_row[kTile];
  int expert, row0, row_end;
  if (!tile_home(offsets, tiles, E, blockIdx.y, expert, row0, row_end)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * GBN;
  if (tid < kTile) {
    const int row = row0 + tid;
    a_row[tid] = row < row_end ? (pair_of_row ? pair_of_row[row] / pairs_per_token : row) : -1;
  }
  __syncthreads();
  const size_t w_rows = GLU ? 2 * (size_t)N : (size_t)N;
  const TW* We = W + (size_t)expert * w_rows * K;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {}, acu[GLU ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < K; k0 += GBK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / GBK, c = idx % GBK;
      const int k = k0 + c;
      const int ar = a_row[r];
      As[c][r] = (ar >= 0 && k < K) ? to_float(A[(size_t)ar * lda + k]) : 0.f;
      const int f = n0 + r;
      if (GLU) {
        const size_t gr = interleaved ? (size_t)(f / 8) * 16 + f % 8 : (size_t)f;
        const size_t ur = interleaved ? gr + 8 : (size_t)N + f;
        Ws[c][r] = (f < N && k < K) ? to_float(We[gr * K + k]) : 0.f;
        Us[c][r] = (f < N && k < K) ? to_float(We[ur * K + k]) : 0.f;
      } else {
        Ws[c][r] = (f < N && k < K) ? to_float(We[(size_t)f * K + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GBK; ++kk) {
      float a[4], w[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[kk][tm + i];
        w[i] = Ws[kk][tn + i];
        if (GLU) u[i] = Us[kk][tn + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (GLU) acu[GLU ? i : 0][j] = fmaf(a[i], u[j], acu[GLU ? i : 0][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = row0 + tm + i;
    if (row >= row_end) continue;
    const float ws = (GLU && pair_scale) ? pair_scale[pair_of_row ? pair_of_row[row] : row] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      const float v = GLU ? clamped_glu(acc[i][j] * ws, acu[GLU ? i : 0][j] * ws, limit, alpha)
                          : plain_activation(acc[i][j], act);
      C[(size_t)row * ldc + n] = from_float<TO>(v);
    }
  }
}

// ---- the grouped products on bfloat16 tensor cores (mma.sync m16n8k16, float32 sums) -------------------------------
// A block of eight warps takes one tile of kTile rows of one expert and MBN weight rows, and walks K in slabs
// of MBK through a ring of cp.async stages (rows of A gathered by the pair's token).  Warps lie 2 x 4 over the
// tile: 32 rows x 32 weight rows each.  GLU: the weight rows come in blocks of 16 (8 gate rows, then the 8 up
// rows of the same features), so a thread that holds a gate sum in one 8-column tile holds the up sum of the
// same feature and row in the next tile, and the activation needs no exchange: C gets MBN / 2 features a block.
constexpr int MBN = 128, MBK = 32, MPAD = 8, MSTAGES = 3;

__device__ __forceinline__ void moe_ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void moe_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void moe_cp_async_16(void* dst, const void* src, bool full) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = full ? 16 : 0;                               // 0: sixteen zero bytes, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}

template <typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_grouped_mma_kernel(const bf16* __restrict__ A, long long lda, const int* __restrict__ pair_of_row, int pairs_per_token,
                       const bf16* __restrict__ W, TO* __restrict__ C, long long ldc, const int* __restrict__ offsets,
                       const int* __restrict__ tiles, int E, int NW, int K, float limit, float alpha,
                       const float* __restrict__ pair_scale, int act) {
  pdl_wait();
  pdl_trigger();
  // NW: weight rows per expert (twice the features when GLU)
  __shared__ __align__(16) bf16 As[MSTAGES][kTile][MBK + MPAD];
  __shared__ __align__(16) bf16 Ws[MSTAGES][MBN][MBK + MPAD];
  __shared__ int a_row[kTile];
  int expert, row0, row_end;
  if (!tile_home(offsets, tiles, E, blockIdx.y, expert, row0, row_end)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 2, wn = warp & 3;                  // the warp's 32 rows and 32 weight rows of the tile
  const int n0 = blockIdx.x * MBN;
  if (tid < kTile) {
    const int row = row0 + tid;
    a_row[tid] = row < row_end ? (pair_of_row ? pair_of_row[row] / pairs_per_token : row) : -1;
  }
  __syncthreads();
  const bf16* We = W + (size_t)expert * NW * K;
  // a thread's copies of a stage: one 16-byte piece of A (64 rows x 4 pieces), two of W (128 rows x 4 pieces)
  const int ar = tid >> 2, ac = (tid & 3) * 8;
  const int a_src = a_row[ar];
  auto fetch = [&](int k0, int st) {
    moe_cp_async_16(&As[st][ar][ac], A + (size_t)(a_src < 0 ? 0 : a_src) * lda + k0 + ac, a_src >= 0 && k0 + ac < K);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int wr = ar + i * 64, n = n0 + wr;
      moe_cp_async_16(&Ws[st][wr][ac], We + (size_t)(n < NW ? n : 0) * K + k0 + ac, n < NW && k0 + ac < K);
    }
    asm volatile("cp.async.commit_group;" ::);
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  const int slabs = (K + MBK - 1) / MBK;
  for (int s = 0; s < MSTAGES - 1; ++s) {
    if (s < slabs) fetch(s * MBK, s);
    else asm volatile("cp.async.commit_group;" ::);
  }
  for (int s = 0; s < slabs; ++s) {
    asm volatile("cp.async.wait_group %0;" ::"n"(MSTAGES - 2));
    __syncthreads();                                        // slab s has landed; the stage of slab s - 1 is free
    if (s + MSTAGES - 1 < slabs) fetch((s + MSTAGES - 1) * MBK, (s + MSTAGES - 1) % MSTAGES);
    else asm volatile("cp.async.commit_group;" ::);
    const int st = s % MSTAGES;
#pragma unroll
    for (int kk = 0; kk < MBK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        moe_ldmatrix_x4(a[i], &As[st][wm * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int j2 = 0; j2 < 2; ++j2) {
        uint32_t b[4];
        moe_ldmatrix_x4(b, &Ws[st][wn * 32 + j2 * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          moe_mma_bf16(acc[i][2 * j2], a[i], b[0], b[1]);
          moe_mma_bf16(acc[i][2 * j2 + 1], a[i], b[2], b[3]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row0 + wm * 32 + i * 16 + (lane >> 2) + 8 * half;
      if (row >= row_end) continue;
      if (GLU) {
        const float ws = pair_scale ? pair_scale[pair_of_row ? pair_of_row[row] : row] : 1.f;
#pragma unroll
        for (int j2 = 0; j2 < 2; ++j2)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int f = (n0 + wn * 32 + j2 * 16) / 2 + (lane & 3) * 2 + c;
            if (2 * f < NW)
              C[(size_t)row * ldc + f] = from_float<TO>(clamped_glu(acc[i][2 * j2][2 * half + c] * ws,
                                                                    acc[i][2 * j2 + 1][2 * half + c] * ws, limit, alpha));
          }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int n = n0 + wn * 32 + j * 8 + (lane & 3) * 2 + c;
            if (n < NW) C[(size_t)row * ldc + n] = from_float<TO>(plain_activation(acc[i][j][2 * half + c], act));
          }
      }
    }
}

// out[t, :] = sum_c weight[t, c] * rows[row_of_pair[t * top + c], :]  (+ shared[t, :]), float32 sums in the order of c;
// weight null: the rows as they are (the weights went into the experts' inputs)
template <typename TR, typename TA>
__global__ void moe_combine_kernel(const TR* __restrict__ rows, long long ldr, const int* __restrict__ row_of_pair,
                                   const float* __restrict__ weight, const TA* __restrict__ shared, TA* __restrict__ out,
                                   int top, int H) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float acc = 0.f;
    for (int c = 0; c < top; ++c) {
      const int row = row_of_pair[(size_t)t * top + c];
      if (row >= 0) acc += (weight ? weight[(size_t)t * top + c] : 1.f) * to_float(rows[(size_t)row * ldr + h]);
    }
    if (shared) acc += to_float(shared[(size_t)t * H + h]);
    out[(size_t)t * H + h] = from_float<TA>(acc);
  }
}

// in [T, ld >= 2 F]: gate in columns [0, F), up in [F, 2 F)  ->  out [T, F]
template <typename TI, typename TA>
__global__ void clamped_glu_kernel(const TI* __restrict__ in, long long ld, TA* __restrict__ out, int F, size_t total,
                                   float limit, float alpha) {
  pdl_wait();
  pdl_trigger();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / F, f = idx - t * F;
    out[idx] = from_float<TA>(clamped_glu(to_float(in[t * ld + f]), to_float(in[t * ld + F + f]), limit, alpha));
  }
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_moe_tile_rows() { return kTile; }

// logits float32 [T, ld >= E]; bias float32 [E] or null; choice int32 [T, top]; weight float32 [T, top]
// scoring 0: weights = softmax over the chosen logits; 1: the logistic of each chosen logit; 2: the softmax over all
// logits, renormalised over the chosen ones, the choice limited to the best `kept` of `groups` equal groups of neighbours
static int routing_ok(const char* what, int E, int top, int scoring, int groups, int kept) {
  if (scoring < 0 || scoring > 2 || groups <= 0 || kept <= 0 || kept > groups || E % groups || groups > 1024 ||
      (groups > 1 && scoring != 2) || (long long)top > (long long)(E / groups) * kept)
    return refuse(ST_BAD_SIZE, "%s: scoring %d, %d experts in %d groups of which %d are kept, top %d", what, scoring, E, groups,
                  kept, top);
  return ST_OK;
}

extern "C" int srlm_moe_route(const float* logits, long long ld, const float* bias, int T, int E, int top, int* choice,
                              float* weight, int scoring, int groups, int kept, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (E <= 0 || top <= 0 || top > E || ld < E || E > 8192)
    return refuse(ST_BAD_SIZE, "moe_route: experts=%d top=%d ld=%lld (at most 8192 experts)", E, top, ld);
  if (int r = routing_ok("moe_route", E, top, scoring, groups, kept)) return r;
  int warps = 4;
  while (warps > 1 && (size_t)warps * E * sizeof(float) > 40 * 1024) warps >>= 1;
  launch_pdl(moe_route_kernel, dim3((T + warps - 1) / warps), dim3(warps * 32), (size_t)warps * E * sizeof(float), stream,
             logits, ld, bias, T, E, top, choice, weight, scoring, groups, kept);
  return launched();
}

// choice int32 [n] (n = tokens x top); offsets, tiles int32 [E + 1]; pair_of_row, row_of_pair int32 [n]
// tile_rows 0: the tiles of the grouped kernels of this file, rows packed.  tile_rows > 0: every expert's rows
// start at a multiple of it; group_of_tile [max_tiles >= (n + E * (tile_rows - 1)) / tile_rows] names each tile's
// expert (-1: none) and pair_of_row has rows_cap >= max_tiles * tile_rows entries (-1: no pair).
// logits (float32 [n / top, ld >= E], with bias [E] or null) given: the kernel routes the tokens first and
// writes choice and weight [n / top, top] itself; offered for E <= 256 (srlm_moe_sort_routes).
extern "C" int srlm_moe_sort_routes(int tokens, int E) { return tokens <= 512 && E <= 256; }

extern "C" int srlm_moe_sort(int* choice, int n, int E, int* offsets, int* tiles, int* pair_of_row,
                             int* row_of_pair, int tile_rows, int* group_of_tile, int max_tiles, int rows_cap,
                             const float* logits, long long ld, const float* bias, int top, float* weight, int scoring,
                             int groups, int kept, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (E <= 0 || E > 4096) return refuse(ST_BAD_SIZE, "moe_sort: experts=%d (at most 4096)", E);
  if (logits)
    if (int r = routing_ok("moe_sort", E, top, scoring, groups, kept)) return r;
  if (logits && (top <= 0 || top > E || n % top || ld < E || !weight || !srlm_moe_sort_routes(n / top, E)))
    return refuse(ST_BAD_SIZE, "moe_sort: routing %d pairs, top=%d of %d experts, ld=%lld", n, top, E, ld);
  const int align = tile_rows > 0;
  if (align && (!group_of_tile || (long long)max_tiles < ((long long)n + (long long)E * (tile_rows - 1)) / tile_rows ||
                rows_cap < max_tiles * tile_rows))
    return refuse(ST_BAD_SIZE, "moe_sort: %d pairs over %d experts in tiles of %d need more than %d tiles, %d rows", n, E,
                  tile_rows, max_tiles, rows_cap);
  const size_t smem = (size_t)(2 * E + 1) * sizeof(int) + (logits ? (size_t)32 * E * sizeof(float) : 0);
  launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, choice, n, E,
             align ? tile_rows : kTile, align, offsets, tiles, pair_of_row, row_of_pair, group_of_tile, max_tiles, rows_cap,
             logits, ld, bias, top, weight, scoring, groups, kept);
  return launched();
}

// xs [rows, K] bfloat16 = the rows of x [tokens, ldx] that pair_of_row names (pair / pairs_per_token), zeros for -1
extern "C" int srlm_moe_gather_rows(const void* x, long long ldx, const int* pair_of_row, int pairs_per_token, void* xs,
                                    int rows, int K, const float* pair_scale, cudaStream_t stream) {
  if (rows <= 0) return ST_OK;
  if (K <= 0 || K % 8 || ldx % 8 || pairs_per_token <= 0 || ((((uintptr_t)x | (uintptr_t)xs) & 15) != 0))
    return refuse(ST_BAD_SIZE, "moe_gather_rows: K=%d ldx=%lld (multiples of 8, 16-byte aligned)", K, ldx);
  const long long total = (long long)rows * (K / 8);
  long long g = (total + 255) / 256;
  launch_pdl(moe_gather_rows_kernel, dim3((unsigned)(g > 148 * 16 ? 148 * 16 : g)), dim3(256), 0, stream, (const bf16*)x, ldx,
             pair_of_row, pairs_per_token, (bf16*)xs, rows, K, pair_scale);
  return launched();
}

// The most tiles a step of n pairs over E experts can have.
static inline int tile_bound(int n, int E) {
  const long long by_rows = (long long)n / kTile + E;      // each expert wastes less than one tile
  return (int)(by_rows < n ? by_rows : n);
}

// glu != 0: W [E, 2 N, K], C [n, N] = the experts' activation; else W [E, N, K], C [n, N] = the product, through the
// exact gelu when act == 1.
// pair_of_row null: row r of A is row r of C (the experts' second product); else A's row is the pair's token.
extern "C" int srlm_moe_grouped_simt(const void* A, int a_dtype, long long lda, const int* pair_of_row, int pairs_per_token,
                                     const void* W, int w_dtype, void* C, int c_dtype, long long ldc, const int* offsets,
                                     const int* tiles, int n, int E, int N, int K, int glu, int interleaved, float limit,
                                     float alpha, const float* pair_scale, int act, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (E <= 0 || N <= 0 || K <= 0 || lda < K || ldc < N || (pair_of_row && pairs_per_token <= 0) ||
      (glu && interleaved && N % 8))
    return refuse(ST_BAD_SIZE, "moe_grouped: experts=%d N=%d K=%d lda=%lld ldc=%lld", E, N, K, lda, ldc);
  const int bound = tile_bound(n, E);
  if (bound > 65535) return refuse(ST_BAD_SIZE, "moe_grouped: %d pairs over %d experts exceed 65535 tiles", n, E);
  dim3 grid((N + GBN - 1) / GBN, bound);
#define SRLM_GROUPED(TA, TW, TO)                                                                                      \
  do {                                                                                                                \
    if (glu) launch_pdl(moe_grouped_simt_kernel<TA, TW, TO, true>, grid, dim3(256), 0, stream, (const TA*)A, lda,    \
                        pair_of_row, pairs_per_token, (const TW*)W, (TO*)C, ldc, offsets, tiles, E, N, K, interleaved, \
                        limit, alpha, pair_scale, act);                                                               \
    else launch_pdl(moe_grouped_simt_kernel<TA, TW, TO, false>, grid, dim3(256), 0, stream, (const TA*)A, lda,       \
                    pair_of_row, pairs_per_token, (const TW*)W, (TO*)C, ldc, offsets, tiles, E, N, K, interleaved,    \
                    limit, alpha, pair_scale, act);                                                                   \
  } while (0)
  if (a_dtype == DT_F32 && w_dtype == DT_F32 && c_dtype == DT_F32) SRLM_GROUPED(float, float, float);
  else if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && c_dtype == DT_BF16) SRLM_GROUPED(bf16, bf16, bf16);
  else if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && c_dtype == DT_F32) SRLM_GROUPED(bf16, bf16, float);
  else return refuse(ST_BAD_DTYPE, "moe_grouped: dtypes (%d, %d) -> %d are not offered", a_dtype, w_dtype, c_dtype);
#undef SRLM_GROUPED
  return launched();
}

// rows [n, ldr] (float32 or the activation dtype); shared [T, H] in the activation dtype or null; out [T, H]
extern "C" int srlm_moe_combine(const void* rows, int rows_dtype, long long ldr, const int* row_of_pair,
                                const float* weight, const void* shared, void* out, int act_dtype, int T, int top, int H,
                                cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (top <= 0 || H <= 0 || ldr < H) return refuse(ST_BAD_SIZE, "moe_combine: top=%d H=%d ldr=%lld", top, H, ldr);
  int block = 32;
  while (block < 256 && block < H) block <<= 1;
#define SRLM_COMBINE(TR, TA)                                                                                   \
  launch_pdl(moe_combine_kernel<TR, TA>, dim3(T), dim3(block), 0, stream, (const TR*)rows, ldr, row_of_pair,  \
             weight, (const TA*)shared, (TA*)out, top, H)
  if (rows_dtype == DT_F32 && act_dtype == DT_F32) SRLM_COMBINE(float, float);
  else if (rows_dtype == DT_F32 && act_dtype == DT_BF16) SRLM_COMBINE(float, bf16);
  else if (rows_dtype == DT_BF16 && act_dtype == DT_BF16) SRLM_COMBINE(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "moe_combine: rows dtype %d with activation dtype %d", rows_dtype, act_dtype);
#undef SRLM_COMBINE
  return launched();
}

// in [T, ld >= 2 F] (float32 or the activation dtype): gate columns, then up columns; out [T, F]
extern "C" int srlm_clamped_glu(const void* in, int in_dtype, long long ld, void* out, int out_dtype, int T, int F,
                                float limit, float alpha, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (F <= 0 || ld < 2ll * F) return refuse(ST_BAD_SIZE, "clamped_glu: F=%d ld=%lld", F, ld);
  const size_t total = (size_t)T * F;
  size_t g = (total + 255) / 256;
  const int grid = (int)(g > 148 * 16 ? 148 * 16 : g);
#define SRLM_GLU(TI, TA) launch_pdl(clamped_glu_kernel<TI, TA>, dim3(grid), dim3(256), 0, stream, (const TI*)in, ld, (TA*)out, F, total, limit, alpha)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) SRLM_GLU(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) SRLM_GLU(float, bf16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) SRLM_GLU(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "clamped_glu: input dtype %d with output dtype %d", in_dtype, out_dtype);
#undef SRLM_GLU
  return launched();
}

// The same products on bfloat16 tensor cores: K a multiple of 8, 16-byte aligned operands; with glu the weight
// rows interleaved in blocks of 16 (8 gate rows, 8 up rows) and N (features) a multiple of 8.
extern "C" int srlm_moe_grouped_mma_takes(int N, int K, int glu) { return K > 0 && K % 8 == 0 && N > 0 && (!glu || N % 8 == 0); }

extern "C" int srlm_moe_grouped_mma(const void* A, long long lda, const int* pair_of_row, int pairs_per_token, const void* W,
                                    void* C, int c_dtype, long long ldc, const int* offsets, const int* tiles, int n, int E,
                                    int N, int K, int glu, float limit, float alpha, const float* pair_scale, int act,
                                    cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (E <= 0 || !srlm_moe_grouped_mma_takes(N, K, glu) || lda < K || lda % 8 || ldc < N || (pair_of_row && pairs_per_token <= 0))
    return refuse(ST_BAD_SIZE, "moe_grouped_mma: experts=%d N=%d K=%d lda=%lld ldc=%lld", E, N, K, lda, ldc);
  if ((((uintptr_t)A | (uintptr_t)W) & 15) != 0) return refuse(ST_BAD_ALIGN, "moe_grouped_mma: operands must be 16-byte aligned");
  const int bound = tile_bound(n, E);
  if (bound > 65535) return refuse(ST_BAD_SIZE, "moe_grouped_mma: %d pairs over %d experts exceed 65535 tiles", n, E);
  const int NW = glu ? 2 * N : N;
  dim3 grid((NW + MBN - 1) / MBN, bound);
#define SRLM_GROUPED_MMA(TO, G)                                                                                          \
  launch_pdl(moe_grouped_mma_kernel<TO, G>, grid, dim3(256), 0, stream, (const bf16*)A, lda, pair_of_row, pairs_per_token, \
             (const bf16*)W, (TO*)C, ldc, offsets, tiles, E, NW, K, limit, alpha, pair_scale, act)
  if (c_dtype == DT_BF16 && glu) SRLM_GROUPED_MMA(bf16, true);
  else if (c_dtype == DT_F32 && glu) SRLM_GROUPED_MMA(float, true);
  else if (c_dtype == DT_BF16) SRLM_GROUPED_MMA(bf16, false);
  else if (c_dtype == DT_F32) SRLM_GROUPED_MMA(float, false);
  else return refuse(ST_BAD_DTYPE, "moe_grouped_mma: output dtype %d", c_dtype);
#undef SRLM_GROUPED_MMA
  return launched();
}
