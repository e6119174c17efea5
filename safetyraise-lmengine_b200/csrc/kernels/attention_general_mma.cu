// The attention of attention_general.cu on bfloat16 tensor cores (mma.sync m16n8k16, float32 sums),
// for steps with many rows (prompts and their portions): keys of dk and values of dv elements, values
// optionally read from the keys' leading part, an optional sink per head.
//
// A block of four warps takes 64 rows (tokens x query heads of one KV head) of one entry and one slab of
// DVT = 64 or 128 value columns, and walks the keys in tiles of 64: S = Q K^T over the whole key size, the
// softmax in registers (float32), O += P V for the block's slab.  A wide value (a latent of 512) is cut
// into slabs with a block each, every block forming S again: the sums of 64 rows x 512 columns do not
// fit a block's registers, and S costs less on tensor cores than it did in float32 arithmetic.
// Queries arrive as float32 and are rounded to bfloat16 as they enter shared memory.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int kMmaRows = 64, kMmaKeys = 64, kMmaWarps = 4, kPad = 8;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool full) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = full ? 16 : 0;                               // 0: sixteen zero bytes, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

template <typename TO, int NT>       // NT: 8-column tiles of the block's slab of values (8 or 16)
__global__ void __launch_bounds__(kMmaWarps * 32)
paged_attention_general_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                                   const bf16* __restrict__ v_cache, TO* __restrict__ out,
                                   const int* __restrict__ block_table, int table_stride,
                                   const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                                   const float* __restrict__ sinks, int nq, int nkv, int dk, int dv, int page_size,
                                   float scale, int window, int nbuf, const bf16* __restrict__ kv_rows,
                                   long long ld_rows, const int* __restrict__ cu_kv, int dim_rows, int v_off,
                                   int page_skip, ScoreMods mods, HeadGate gate) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  // kv_rows != null: every query head has keys and values of its own (nkv = nq), formed for this step in
  // kv_rows, row cu_kv[e] + j for key j of entry e: the key's first dim_rows elements at column kvh * dim_rows,
  // its values at column v_off + kvh * dv.  The key's other dk - dim_rows elements are shared by the heads and
  // read from the pages (one KV head, rows of page_skip + dk - dim_rows elements, behind the first page_skip).
  constexpr int DVT = 8 * NT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int slabs = dv / DVT;
  const int e = blockIdx.z, kvh = blockIdx.y / slabs, slab = blockIdx.y % slabs;
  const int G = nq / nkv;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0, kv_len = kv_lens[e];
  const int rows = q_len * G;
  const int r0 = blockIdx.x * kMmaRows;
  if (r0 >= rows) return;
  const int ks = dk + kPad;                                 // row strides in elements; rows stay 16-byte aligned
  const bool own_values = v_cache || kv_rows;               // a tile of values of their own, not the keys' leading part
  const int vs = own_values ? DVT + kPad : ks;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [64][dk + 8]
  // nbuf = 2 when two tiles of keys (and values) fit beside the queries: the next tile is fetched (cp.async)
  // while this one is worked on; nbuf = 1: fetched, waited for, worked on
  bf16* k_s = q_s + kMmaRows * ks;                          // [nbuf][64][dk + 8]
  bf16* v_s = own_values ? k_s + nbuf * kMmaKeys * ks : k_s + slab * DVT;   // [nbuf][64][DVT + 8], or the slab's columns of the keys
  const int k_tile = kMmaKeys * ks, v_tile = own_values ? kMmaKeys * vs : k_tile;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = kv_len - q_len;
  const int* table = block_table + (size_t)e * table_stride;

  for (int idx = tid; idx < kMmaRows * dk; idx += blockDim.x) {
    const int r = idx / dk, d = idx - r * dk, row = r0 + r;
    const float v = row < rows ? q[((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dk + d] : 0.f;
    q_s[r * ks + d] = __float2bfloat16_rn(v);
  }

  // a thread's two rows of its warp's 16: lane / 4 and lane / 4 + 8
  float m[2], l[2], row_scale[2], pen_w[2], pen_r[2];
  int pos[2], first[2];
  const bool penalised = mods.pen_weight != nullptr;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * i;
    const bool live = row < rows;
    pos[i] = live ? start + row / G : -1;
    first[i] = (window > 0 && live) ? max(0, pos[i] - window + 1) : 0;
    const int h = kvh * G + (live ? row % G : 0);
    row_scale[i] = mods.head_scale ? scale * mods.head_scale[h] : scale;
    pen_w[i] = penalised ? mods.pen_weight[h] : 0.f;
    pen_r[i] = penalised ? mods.pen_rate[h] : 0.f;
    m[i] = sinks ? sinks[h] : -CUDART_INF_F;
    l[i] = sinks ? 1.f : 0.f;
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  const int last_row = min(rows, r0 + kMmaRows) - 1;
  const int max_pos = start + last_row / G, min_pos = start + r0 / G;
  const int first_key = window > 0 ? max(0, min_pos - window + 1) : 0;
  const int kvec = dk / 8, vvec = DVT / 8;

  const long long row0 = kv_rows ? (long long)cu_kv[e] : 0;       // where key 0 would lie: negative when the first keys were not gathered
  const int page_width = page_skip + dk - dim_rows;
  auto fetch = [&](int jb, int buf) {
    for (int idx = tid; idx < kMmaKeys * kvec; idx += blockDim.x) {
      const int jj = idx / kvec, c = idx - jj * kvec, j = jb + jj;
      const bool there = j >= first_key && j <= max_pos;     // pages before a window's first key may be given back
      const bf16* src = k_cache;
      if (there && kv_rows) {
        if (c * 8 < dim_rows) {
          src = kv_rows + (size_t)(row0 + j) * ld_rows + (size_t)kvh * dim_rows + c * 8;
        } else {
          const size_t rowi = (size_t)table[j / page_size] * page_size + (j % page_size);
          src = k_cache + rowi * page_width + page_skip + (c * 8 - dim_rows);
        }
      } else if (there) {
        const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
        src = k_cache + rowi * dk + c * 8;
      }
      cp_async_16(k_s + buf * k_tile + jj * ks + c * 8, src, there);
    }
    if (v_cache || kv_rows) {
      for (int idx = tid; idx < kMmaKeys * vvec; idx += blockDim.x) {
        const int jj = idx / vvec, c = idx - jj * vvec, j = jb + jj;
        const bool there = j >= first_key && j <= max_pos;     // pages before a window's first key may be given back
        const bf16* src = k_cache;
        if (there && kv_rows) {
          src = kv_rows + (size_t)(row0 + j) * ld_rows + v_off + (size_t)kvh * dv + slab * DVT + c * 8;
        } else if (there) {
          const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
          src = v_cache + rowi * dv + slab * DVT + c * 8;
        }
        cp_async_16(v_s + buf * v_tile + jj * vs + c * 8, src, there);
      }
    }
    cp_async_commit();
  };
  const int jb0 = (first_key / kMmaKeys) * kMmaKeys;
  if (nbuf == 2 && jb0 <= max_pos) fetch(jb0, 0);
  int buf = 0;
  for (int jb = jb0; jb <= max_pos; jb += kMmaKeys) {
    if (nbuf == 2) {
      if (jb + kMmaKeys <= max_pos) {
        fetch(jb + kMmaKeys, buf ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
    } else {
      __syncthreads();                                      // the tile is no longer read
      fetch(jb, 0);
      cp_async_wait<0>();
    }
    __syncthreads();

    // S = Q K^T: 16 rows x 64 keys a warp
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
    const bf16* qa = q_s + (warp * 16 + (lane & 15)) * ks + (lane >> 4) * 8;
    const bf16* kb = k_s + buf * k_tile + ((lane & 7) + (lane >> 4) * 8) * ks + ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < dk; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, qa + k0);
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t b[4];
        ldmatrix_x4(b, kb + n2 * 16 * ks + k0);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }

    // softmax of this tile, in registers
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = jb + n * 8 + (lane & 3) * 2 + c;
          const bool valid = j <= pos[i] && j >= first[i];
          float v = -CUDART_INF_F;
          if (valid) {
            v = capped_score(s[n][2 * i + c] * row_scale[i], mods.softcap);
            if (penalised) v -= distance_penalty(pen_w[i], pen_r[i], pos[i] - j);
          }
          s[n][2 * i + c] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[i], mx);
      float alpha = 1.f, sum = 0.f;
      if (m_new != -CUDART_INF_F) {
        alpha = expf(m[i] - m_new);
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float p = expf(s[n][2 * i + c] - m_new);       // exp(-inf) = 0 for masked keys
            s[n][2 * i + c] = p;
            sum += p;
          }
      } else {
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][2 * i] = s[n][2 * i + 1] = 0.f;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[i] = l[i] * alpha + sum;
      m[i] = m_new;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][2 * i] *= alpha;
        o[n][2 * i + 1] *= alpha;
      }
    }

    // O += P V for the slab
    const bf16* vb = v_s + buf * v_tile + (lane & 15) * vs + (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vb + kk * 16 * vs + n2 * 16);
        mma_bf16(o[2 * n2], a, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
      }
    }
    if (nbuf == 2) {
      __syncthreads();                                      // before the next fetch goes into this tile's twin
      buf ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + warp * 16 + (lane >> 2) + 8 * i;
    if (row >= rows) continue;
    const float inv = head_gate_of(gate, (size_t)(t0 + row / G), kvh * G + row % G) / l[i];
    TO* dst = out + ((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dv + slab * DVT + (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      dst[n * 8] = from_float<TO>(o[n][2 * i] * inv);
      dst[n * 8 + 1] = from_float<TO>(o[n][2 * i + 1] * inv);
    }
  }
}

// ---- decode steps: entries of at most 16 rows -------------------------------------------------------------
// A block takes one slice of an entry's keys for one KV head.  Its four warps walk the same tiles of 32 keys
// (fetched with cp.async, two tiles in flight) and all form the same S and the same softmax for the 16 rows;
// each warp owns a quarter of the value columns (NTW tiles of 8), so a wide value needs no second pass over
// the keys, which is what a decode step is bound by.  nsplit > 1: the slices' unnormalised sums go to
// part_o / part_ml (the entry's rows padded to whole tiles of 16 per slice) and attention_general.cu's merge
// kernel adds them.  An entry of more than 16 rows (many query heads per KV head, or a few tokens) is several
// blocks, each walking the slice again: the second reading comes from L2.
constexpr int kDecKeys = 32;

template <typename TO, int NTW>
__global__ void __launch_bounds__(kMmaWarps * 32)
paged_attention_general_decode_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                                      const bf16* __restrict__ v_cache, TO* __restrict__ out,
                                      const int* __restrict__ block_table, int table_stride,
                                      const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                                      const float* __restrict__ sinks, int nq, int nkv, int dk, int dv,
                                      int page_size, float scale, int window, int nsplit, int kv_chunk,
                                      float* __restrict__ part_o, float* __restrict__ part_ml, int row_tiles,
                                      ScoreMods mods, HeadGate gate) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int e = blockIdx.z, kvh = blockIdx.y / row_tiles, slice = blockIdx.x;
  const int r0 = (blockIdx.y % row_tiles) * 16;             // the block's 16 rows of the entry's q_len * G
  const int G = nq / nkv;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0, kv_len = kv_lens[e];
  const int rows = q_len * G;
  if (r0 >= rows) return;
  const int ks = dk + kPad, vs = v_cache ? dv + kPad : ks;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);            // [16][dk + 8]
  bf16* k_s = q_s + 16 * ks;                                // [2][32][dk + 8]
  bf16* v_s = v_cache ? k_s + 2 * kDecKeys * ks : k_s;      // [2][32][dv + 8], or the keys
  const int k_tile = kDecKeys * ks, v_tile = v_cache ? kDecKeys * vs : k_tile;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = kv_len - q_len;
  const int* table = block_table + (size_t)e * table_stride;

  for (int idx = tid; idx < 16 * dk; idx += blockDim.x) {
    const int r = idx / dk, d = idx - r * dk, row = r0 + r;
    const float v = row < rows ? q[((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dk + d] : 0.f;
    q_s[r * ks + d] = __float2bfloat16_rn(v);
  }
  float m[2], l[2], row_scale[2], pen_w[2], pen_r[2];
  int pos[2], first[2];
  const bool penalised = mods.pen_weight != nullptr;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + (lane >> 2) + 8 * i;
    const bool live = row < rows;
    pos[i] = live ? start + row / G : -1;
    first[i] = (window > 0 && live) ? max(0, pos[i] - window + 1) : 0;
    const int h = kvh * G + (live ? row % G : 0);
    row_scale[i] = mods.head_scale ? scale * mods.head_scale[h] : scale;
    pen_w[i] = penalised ? mods.pen_weight[h] : 0.f;
    pen_r[i] = penalised ? mods.pen_rate[h] : 0.f;
    const bool with_sink = sinks && slice == 0;             // the sink counts once
    m[i] = with_sink ? sinks[kvh * G + (live ? row % G : 0)] : -CUDART_INF_F;
    l[i] = with_sink ? 1.f : 0.f;
  }
  float o[NTW][4];
#pragma unroll
  for (int n = 0; n < NTW; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;

  const int max_pos = start + (min(rows, r0 + 16) - 1) / G;
  int first_key = window > 0 ? max(0, start + r0 / G - window + 1) : 0;
  int last_key = max_pos;
  if (nsplit > 1) {
    // the slices lie over the keys the rows can see: from the key tile that holds the window's first key
    const int base = (first_key / kDecKeys) * kDecKeys;
    first_key = max(first_key, base + slice * kv_chunk);
    last_key = min(last_key, base + (slice + 1) * kv_chunk - 1);
  }
  const int jb0 = (first_key / kDecKeys) * kDecKeys;
  const int kvec = dk / 8, vvec = dv / 8;
  auto fetch = [&](int jb, int buf) {
    for (int idx = tid; idx < kDecKeys * kvec; idx += blockDim.x) {
      const int jj = idx / kvec, c = idx - jj * kvec, j = jb + jj;
      const bool there = j >= first_key && j <= last_key;
      const size_t rowi = there ? ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size) : 0;
      cp_async_16(k_s + buf * k_tile + jj * ks + c * 8, k_cache + rowi * dk + c * 8, there);
    }
    if (v_cache) {
      for (int idx = tid; idx < kDecKeys * vvec; idx += blockDim.x) {
        const int jj = idx / vvec, c = idx - jj * vvec, j = jb + jj;
        const bool there = j >= first_key && j <= last_key;
        const size_t rowi = there ? ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size) : 0;
        cp_async_16(v_s + buf * v_tile + jj * vs + c * 8, v_cache + rowi * dv + c * 8, there);
      }
    }
    cp_async_commit();
  };
  if (jb0 <= last_key) fetch(jb0, 0);
  int buf = 0;
  for (int jb = jb0; jb <= last_key; jb += kDecKeys, buf ^= 1) {
    if (jb + kDecKeys <= last_key) {
      fetch(jb + kDecKeys, buf ^ 1);                        // the tile after this one, into the other buffer
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
    const bf16* qa = q_s + (lane & 15) * ks + (lane >> 4) * 8;
    const bf16* kb = k_s + buf * k_tile + ((lane & 7) + (lane >> 4) * 8) * ks + ((lane >> 3) & 1) * 8;
    for (int k0 = 0; k0 < dk; k0 += 16) {
      uint32_t a[4];
      ldmatrix_x4(a, qa + k0);
#pragma unroll
      for (int n2 = 0; n2 < 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4(b, kb + n2 * 16 * ks + k0);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = jb + n * 8 + (lane & 3) * 2 + c;
          const bool valid = j <= pos[i] && j >= first[i] && j >= first_key && j <= last_key;
          float v = -CUDART_INF_F;
          if (valid) {
            v = capped_score(s[n][2 * i + c] * row_scale[i], mods.softcap);
            if (penalised) v -= distance_penalty(pen_w[i], pen_r[i], pos[i] - j);
          }
          s[n][2 * i + c] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[i], mx);
      float alpha = 1.f, sum = 0.f;
      if (m_new != -CUDART_INF_F) {
        alpha = expf(m[i] - m_new);
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float p = expf(s[n][2 * i + c] - m_new);
            s[n][2 * i + c] = p;
            sum += p;
          }
      } else {
#pragma unroll
        for (int n = 0; n < 4; ++n) s[n][2 * i] = s[n][2 * i + 1] = 0.f;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[i] = l[i] * alpha + sum;
      m[i] = m_new;
#pragma unroll
      for (int n = 0; n < NTW; ++n) {
        o[n][2 * i] *= alpha;
        o[n][2 * i + 1] *= alpha;
      }
    }
    const bf16* vb = v_s + buf * v_tile + (lane & 15) * vs + warp * (NTW * 8) + (lane >> 4) * 8;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int n2 = 0; n2 < NTW / 2; ++n2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vb + kk * 16 * vs + n2 * 16);
        mma_bf16(o[2 * n2], a, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();                                         // before the next fetch overwrites this buffer's twin
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + (lane >> 2) + 8 * i;
    if (row >= rows) continue;
    const int col0 = warp * (NTW * 8) + (lane & 3) * 2;
    if (nsplit > 1) {
      const size_t slab = (((size_t)e * nkv + kvh) * nsplit + slice) * (16 * row_tiles) + row;
#pragma unroll
      for (int n = 0; n < NTW; ++n) {
        part_o[slab * dv + col0 + n * 8] = o[n][2 * i];
        part_o[slab * dv + col0 + n * 8 + 1] = o[n][2 * i + 1];
      }
      if (warp == 0 && (lane & 3) == 0) {
        part_ml[slab * 2] = m[i];
        part_ml[slab * 2 + 1] = l[i];
      }
    } else {
      const float inv = head_gate_of(gate, (size_t)(t0 + row / G), kvh * G + row % G) / l[i];
      TO* dst = out + ((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dv + col0;
#pragma unroll
      for (int n = 0; n < NTW; ++n) {
        dst[n * 8] = from_float<TO>(o[n][2 * i] * inv);
        dst[n * 8 + 1] = from_float<TO>(o[n][2 * i + 1] * inv);
      }
    }
  }
}

template <typename TO, int NT>
static int launch_mma(dim3 grid, size_t smem, cudaStream_t stream, const float* q, const void* k_cache,
                      const void* v_cache, void* out, const int* block_table, int table_stride, const int* cu_q,
                      const int* kv_lens, const float* sinks, int nq, int nkv, int dk, int dv, int page_size,
                      float scale, int window, int nbuf, const bf16* kv_rows = nullptr, long long ld_rows = 0,
                      const int* cu_kv = nullptr, int dim_rows = 0, int v_off = 0, int page_skip = 0,
                      ScoreMods mods = ScoreMods{nullptr, nullptr, nullptr, 0.f}, HeadGate gate = HeadGate{nullptr, 0}) {
  auto kern = paged_attention_general_mma_kernel<TO, NT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(kern, dim3(grid), dim3(kMmaWarps * 32), smem, stream, q, (const bf16*)k_cache, (const bf16*)v_cache, (TO*)out, block_table,
                                               table_stride, cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size, scale,
                                               window, nbuf, kv_rows, ld_rows, cu_kv, dim_rows, v_off, page_skip, mods, gate);
  return launched();
}

}  // namespace srlm

using namespace srlm;

// Whether the tensor-core form takes these sizes: key size a multiple of 16, value size a multiple of 64,
// and two tiles of 64 rows of the key size within a block's shared memory.
extern "C" int srlm_attention_general_mma_takes(int dk, int dv, int values_from_keys) {
  if (dk <= 0 || dv <= 0 || dk % 16 || dv % 64 || (values_from_keys && dv > dk)) return 0;
  const size_t slab = dv % 128 == 0 ? 128 : 64;
  const size_t smem = (size_t)2 * kMmaRows * (dk + kPad) * 2 + (values_from_keys ? 0 : kMmaKeys * (slab + kPad) * 2);
  return smem <= 220 * 1024 ? 1 : 0;
}

// The contract of srlm_paged_attention_general for a bfloat16 cache, without key slices.
extern "C" int srlm_paged_attention_general_mma(const float* q, const void* k_cache, const void* v_cache, void* out,
                                                int out_dtype, const int* block_table, int table_stride,
                                                const int* cu_q, const int* kv_lens, const float* sinks,
                                                int n_entries, int max_q_len, int nq, int nkv, int dk, int dv,
                                                int page_size, float scale, int window, const float* head_scale,
                                                const float* pen_weight, const float* pen_rate, float softcap,
                                                const float* gate_logits, long long ld_gate, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return ST_OK;
  const HeadGate gate{gate_logits, ld_gate};
  if ((pen_weight == nullptr) != (pen_rate == nullptr))
    return refuse(ST_BAD_SIZE, "paged_attention_general_mma: a distance penalty needs its weight and its rate");
  const ScoreMods mods{head_scale, pen_weight, pen_rate, softcap};
  if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || !srlm_attention_general_mma_takes(dk, dv, v_cache ? 0 : 1))
    return refuse(ST_BAD_SIZE, "paged_attention_general_mma: nq=%d nkv=%d dk=%d dv=%d page_size=%d (dk a multiple of "
                  "16, dv of 64)", nq, nkv, dk, dv, page_size);
  if ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
    return refuse(ST_BAD_ALIGN, "paged_attention_general_mma: the pools must be 16-byte aligned");
  const int slab = dv % 128 == 0 ? 128 : 64;
  const int G = nq / nkv;
  const long long tiles = ((long long)max_q_len * G + kMmaRows - 1) / kMmaRows;
  const long long y = (long long)nkv * (dv / slab);
  if (n_entries > 65535 || y > 65535) return refuse(ST_BAD_SIZE, "paged_attention_general_mma: %d entries", n_entries);
  dim3 grid((unsigned)tiles, (unsigned)y, (unsigned)n_entries);
  const size_t q_bytes = (size_t)kMmaRows * (dk + kPad) * 2;
  const size_t tile_bytes = (size_t)kMmaKeys * (dk + kPad) * 2 + (v_cache ? (size_t)kMmaKeys * (slab + kPad) * 2 : 0);
  // two tiles in flight when that still leaves room for two blocks an SM
  const int nbuf = q_bytes + 2 * tile_bytes <= 100 * 1024 ? 2 : 1;
  const size_t smem = q_bytes + nbuf * tile_bytes;
#define SRLM_MMA_ARGS grid, smem, stream, q, k_cache, v_cache, out, block_table, table_stride, cu_q, kv_lens, sinks, nq, \
                      nkv, dk, dv, page_size, scale, window, nbuf, nullptr, 0, nullptr, 0, 0, 0, mods, gate
  if (out_dtype == DT_F32) return slab == 128 ? launch_mma<float, 16>(SRLM_MMA_ARGS) : launch_mma<float, 8>(SRLM_MMA_ARGS);
  if (out_dtype == DT_BF16) return slab == 128 ? launch_mma<bf16, 16>(SRLM_MMA_ARGS) : launch_mma<bf16, 8>(SRLM_MMA_ARGS);
#undef SRLM_MMA_ARGS
  return refuse(ST_BAD_DTYPE, "paged_attention_general_mma: output dtype %d", out_dtype);
}

// Decode steps (entries of a few rows each) over a bfloat16 cache: value size 64, 128, 256 or 512, key size
// a multiple of 16.  With nsplit > 1 the caller then runs srlm_attention_general_merge over part_o / part_ml.
extern "C" int srlm_attention_general_decode_takes(int dk, int dv, int values_from_keys) {
  if (dk <= 0 || dk % 16 || (dv != 64 && dv != 128 && dv != 256 && dv != 512) || (values_from_keys && dv > dk)) return 0;
  const size_t smem = (size_t)(16 + 2 * kDecKeys) * (dk + kPad) * 2 + (values_from_keys ? 0 : (size_t)2 * kDecKeys * (dv + kPad) * 2);
  return smem <= 220 * 1024 ? 1 : 0;
}

extern "C" int srlm_paged_attention_general_decode(const float* q, const void* k_cache, const void* v_cache, void* out,
                                                   int out_dtype, const int* block_table, int table_stride,
                                                   const int* cu_q, const int* kv_lens, const float* sinks,
                                                   int n_entries, int max_q_len, int nq, int nkv, int dk, int dv,
                                                   int page_size, float scale, int window, int nsplit, int kv_chunk,
                                                   float* part_o, float* part_ml, const float* head_scale,
                                                   const float* pen_weight, const float* pen_rate, float softcap,
                                                   const float* gate_logits, long long ld_gate, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return ST_OK;
  const HeadGate gate{gate_logits, ld_gate};
  if ((pen_weight == nullptr) != (pen_rate == nullptr))
    return refuse(ST_BAD_SIZE, "paged_attention_general_decode: a distance penalty needs its weight and its rate");
  const ScoreMods mods{head_scale, pen_weight, pen_rate, softcap};
  if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || !srlm_attention_general_decode_takes(dk, dv, v_cache ? 0 : 1))
    return refuse(ST_BAD_SIZE, "paged_attention_general_decode: nq=%d nkv=%d dk=%d dv=%d rows=%d", nq, nkv, dk, dv,
                  max_q_len * (nq / (nkv > 0 ? nkv : 1)));
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && (kv_chunk <= 0 || kv_chunk % kDecKeys || !part_o || !part_ml))
    return refuse(ST_BAD_SIZE, "paged_attention_general_decode: %d slices of %d keys need a workspace", nsplit, kv_chunk);
  if ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0)
    return refuse(ST_BAD_ALIGN, "paged_attention_general_decode: the pools must be 16-byte aligned");
  const int row_tiles = (int)(((long long)max_q_len * (nq / nkv) + 15) / 16);
  if (n_entries > 65535 || (long long)nkv * row_tiles > 65535)
    return refuse(ST_BAD_SIZE, "paged_attention_general_decode: %d entries, %d row tiles", n_entries, row_tiles);
  dim3 grid((unsigned)nsplit, (unsigned)(nkv * row_tiles), (unsigned)n_entries);
  const size_t smem = (size_t)(16 + 2 * kDecKeys) * (dk + kPad) * 2 + (v_cache ? (size_t)2 * kDecKeys * (dv + kPad) * 2 : 0);
#define SRLM_DEC(TO, NTW)                                                                                          \
  do {                                                                                                             \
    auto kern = paged_attention_general_decode_kernel<TO, NTW>;                                                    \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    launch_pdl(kern, dim3(grid), dim3(kMmaWarps * 32), smem, stream, q, (const bf16*)k_cache, (const bf16*)v_cache, (TO*)out,          \
                                                 block_table, table_stride, cu_q, kv_lens, sinks, nq, nkv, dk, dv, \
                                                 page_size, scale, window, nsplit, kv_chunk, part_o, part_ml,      \
                                                 row_tiles, mods, gate);                                           \
  } while (0)
#define SRLM_DEC_SIZES(TO)                                \
  do {                                                    \
    if (dv == 64) SRLM_DEC(TO, 2);                        \
    else if (dv == 128) SRLM_DEC(TO, 4);                  \
    else if (dv == 256) SRLM_DEC(TO, 8);                  \
    else SRLM_DEC(TO, 16);                                \
  } while (0)
  if (out_dtype == DT_F32) SRLM_DEC_SIZES(float);
  else if (out_dtype == DT_BF16) SRLM_DEC_SIZES(bf16);
  else return refuse(ST_BAD_DTYPE, "paged_attention_general_decode: output dtype %d", out_dtype);
#undef SRLM_DEC_SIZES
#undef SRLM_DEC
  return launched();
}

// Prompts of an attention over a cached latent, in the heads' own space: q float32 [T, heads, dim + rot];
// kv_rows bfloat16 [sum of the entries' contexts, ld_rows]: per row the heads' unrotated keys (heads x dim) and,
// from column v_off, their values (heads x dv); pages: one KV head, rows [latent (rank) | rotated key part (rot)].
// Row cu_kv[e] + j holds key j of entry e; keys that no row of the step sees (behind the window) need no row, so cu_kv[e]
// may be negative.  window > 0: a query sees itself and the window - 1 keys before it.
extern "C" int srlm_latent_prefill_attention_takes(int dim, int rot, int dv, int rank) {
  return dim > 0 && rot >= 0 && dim % 8 == 0 && rot % 8 == 0 && rank % 8 == 0 && (dim + rot) % 16 == 0 && dv % 64 == 0 &&
         srlm_attention_general_mma_takes(dim + rot, dv, 0);
}

extern "C" int srlm_latent_prefill_attention(const float* q, const void* pages, const void* kv_rows, long long ld_rows,
                                             const int* cu_kv, void* out, int out_dtype, const int* block_table,
                                             int table_stride, const int* cu_q, const int* kv_lens, int n_entries,
                                             int max_q_len, int heads, int dim, int rot, int dv, int rank, int v_off,
                                             int page_size, float scale, int window, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return ST_OK;
  if (heads <= 0 || page_size <= 0 || !kv_rows || !cu_kv || !srlm_latent_prefill_attention_takes(dim, rot, dv, rank) ||
      ld_rows % 8 || v_off % 8 || ld_rows < v_off + (long long)heads * dv)
    return refuse(ST_BAD_SIZE, "latent_prefill_attention: heads=%d dim=%d rot=%d dv=%d rank=%d ld=%lld v_off=%d", heads, dim,
                  rot, dv, rank, ld_rows, v_off);
  if ((((uintptr_t)pages | (uintptr_t)kv_rows) & 15) != 0)
    return refuse(ST_BAD_ALIGN, "latent_prefill_attention: pages and rows must be 16-byte aligned");
  const int dk = dim + rot, slab = dv % 128 == 0 ? 128 : 64;
  const long long tiles = ((long long)max_q_len + kMmaRows - 1) / kMmaRows, y = (long long)heads * (dv / slab);
  if (n_entries > 65535 || y > 65535) return refuse(ST_BAD_SIZE, "latent_prefill_attention: %d entries", n_entries);
  dim3 grid((unsigned)tiles, (unsigned)y, (unsigned)n_entries);
  const size_t q_bytes = (size_t)kMmaRows * (dk + kPad) * 2;
  const size_t tile_bytes = (size_t)kMmaKeys * (dk + kPad) * 2 + (size_t)kMmaKeys * (slab + kPad) * 2;
  const int nbuf = q_bytes + 2 * tile_bytes <= 100 * 1024 ? 2 : 1;
  const size_t smem = q_bytes + nbuf * tile_bytes;
#define SRLM_LAT_ARGS grid, smem, stream, q, pages, nullptr, out, block_table, table_stride, cu_q, kv_lens, nullptr, heads, \
                      heads, dk, dv, page_size, scale, window, nbuf, (const bf16*)kv_rows, ld_rows, cu_kv, dim, v_off, rank
  if (out_dtype == DT_F32) return slab == 128 ? launch_mma<float, 16>(SRLM_LAT_ARGS) : launch_mma<float, 8>(SRLM_LAT_ARGS);
  if (out_dtype == DT_BF16) return slab == 128 ? launch_mma<bf16, 16>(SRLM_LAT_ARGS) : launch_mma<bf16, 8>(SRLM_LAT_ARGS);
#undef SRLM_LAT_ARGS
  return refuse(ST_BAD_DTYPE, "latent_prefill_attention: output dtype %d", out_dtype);
}
