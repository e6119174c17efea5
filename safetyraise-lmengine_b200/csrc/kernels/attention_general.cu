// Paged causal attention for heads whose keys and values differ in size, float32 arithmetic.
//
// What it adds to the attention of equal head sizes:
//   * dk (query/key size) and dv (value size) are separate; with no value pool the values ARE the
//     first dv elements of the keys (a cache that holds one latent vector per token serves as both);
//   * an optional sink per query head: one more term exp(sink) in the softmax denominator, with no
//     key and no value behind it;
//   * queries are float32 (they may be the product of a projection folded into them);
//   * optional changes to the scores (ScoreMods in common.cuh): a learned factor per head, a cap by a tanh,
//     and a penalty that grows with the logarithm of the distance between query and key.
//
// A block takes 16 rows (tokens x query heads of one KV head) of one entry and walks the keys in
// blocks of 32 aligned to the start of the sequence; a row's sums depend on its position alone (key
// blocks that a row does not see leave its running maximum, sum and output bit for bit as they were),
// so the result is the same however the tokens were cut into steps or batched.
//
// Beside it: the kernel that adds the projections' biases, mixes the values with those kept from an
// earlier layer and appends keys and values to the pages.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int kRows = 16, kKeys = 32, kWarps = 4, kRowsPerWarp = kRows / kWarps;

template <typename TC, typename TO, int VPL>
__global__ void __launch_bounds__(kWarps * 32)
paged_attention_general_kernel(const float* __restrict__ q, const TC* __restrict__ k_cache,
                               const TC* __restrict__ v_cache, TO* __restrict__ out,
                               const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_q,
                               const int* __restrict__ kv_lens, const float* __restrict__ sinks, int nq, int nkv,
                               int dk, int dv, int page_size, float scale, int window, int nsplit, int kv_chunk,
                               float* __restrict__ part_o, float* __restrict__ part_ml, ScoreMods mods, HeadGate gate) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  extern __shared__ float smem[];
  const int e = blockIdx.z, kvh = blockIdx.y;
  const int G = nq / nkv;
  const int t0 = cu_q[e], q_len = cu_q[e + 1] - t0, kv_len = kv_lens[e];
  const int rows = q_len * G;
  // nsplit > 1 (entries of at most kRows rows): blockIdx.x is a slice of kv_chunk keys, not a row tile;
  // the slices' unnormalised sums go to part_o / part_ml and attention_merge_kernel adds them
  const bool sliced = nsplit > 1;
  const int r0 = sliced ? 0 : blockIdx.x * kRows;
  if (r0 >= rows) return;
  const int ks = dk + 1;                                   // padded key row: lanes read different banks
  float* q_s = smem;                                       // [kRows][dk]
  float* k_s = q_s + kRows * dk;                           // [kKeys][dk + 1]
  float* v_s = v_cache ? k_s + kKeys * ks : k_s;           // [kKeys][dv], or the keys' leading part
  const int vs = v_cache ? dv : ks;
  float* p_s = k_s + kKeys * ks + (v_cache ? kKeys * dv : 0);   // [kRows][kKeys]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int start = kv_len - q_len;                        // position of the entry's first token of this step
  const int* table = block_table + (size_t)e * table_stride;

  for (int idx = tid; idx < kRows * dk; idx += blockDim.x) {
    const int r = idx / dk, d = idx - r * dk, row = r0 + r;
    q_s[idx] = row < rows ? q[((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dk + d] : 0.f;
  }

  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][VPL];
  float row_scale[kRowsPerWarp], pen_w[kRowsPerWarp], pen_r[kRowsPerWarp];
  int pos[kRowsPerWarp], first[kRowsPerWarp];
  const bool penalised = mods.pen_weight != nullptr;
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int row = r0 + warp * kRowsPerWarp + i;
    const bool live = row < rows;
    pos[i] = live ? start + row / G : -1;                  // a row beyond the entry sees no key
    first[i] = (window > 0 && live) ? max(0, pos[i] - window + 1) : 0;
    const int h = kvh * G + (live ? row % G : 0);
    row_scale[i] = mods.head_scale ? scale * mods.head_scale[h] : scale;
    pen_w[i] = penalised ? mods.pen_weight[h] : 0.f;
    pen_r[i] = penalised ? mods.pen_rate[h] : 0.f;
    const bool with_sink = sinks && (!sliced || blockIdx.x == 0);     // the sink counts once
    m[i] = with_sink ? sinks[h] : -CUDART_INF_F;
    l[i] = with_sink ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < VPL; ++c) acc[i][c] = 0.f;
  }
  const int last_row = min(rows, r0 + kRows) - 1;
  const int max_pos = start + last_row / G, min_pos = start + r0 / G;
  int first_key = window > 0 ? max(0, min_pos - window + 1) : 0;
  int last_key = max_pos;
  if (sliced) {                                            // kv_chunk is a multiple of kKeys
    // the slices lie over the keys the rows can see: from the key block that holds the window's first key
    const int base = (first_key / kKeys) * kKeys;
    first_key = max(first_key, base + (int)blockIdx.x * kv_chunk);
    last_key = min(last_key, base + ((int)blockIdx.x + 1) * kv_chunk - 1);
  }

  for (int jb = (first_key / kKeys) * kKeys; jb <= last_key; jb += kKeys) {
    __syncthreads();                                       // the tile of the iteration before is no longer read
    for (int idx = tid; idx < kKeys * dk; idx += blockDim.x) {
      const int jj = idx / dk, d = idx - jj * dk, j = jb + jj;
      float v = 0.f;
      if (j >= first_key && j <= last_key) {               // pages before a window's first key may be given back
        const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
        v = to_float(k_cache[rowi * dk + d]);
      }
      k_s[jj * ks + d] = v;
    }
    if (v_cache) {
      for (int idx = tid; idx < kKeys * dv; idx += blockDim.x) {
        const int jj = idx / dv, d = idx - jj * dv, j = jb + jj;
        float v = 0.f;
        if (j >= first_key && j <= last_key) {               // pages before a window's first key may be given back
          const size_t rowi = ((size_t)table[j / page_size] * nkv + kvh) * page_size + (j % page_size);
          v = to_float(v_cache[rowi * dv + d]);
        }
        v_s[jj * dv + d] = v;
      }
    }
    __syncthreads();

    float dot[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) dot[i] = 0.f;
    const float* kr = k_s + lane * ks;
    const float* qr = q_s + warp * kRowsPerWarp * dk;
    for (int d = 0; d < dk; ++d) {
      const float kv = kr[d];
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) dot[i] += qr[i * dk + d] * kv;
    }
    const int j = jb + lane;
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      const bool valid = j <= pos[i] && j >= first[i];
      float s = -CUDART_INF_F;
      if (valid) {
        s = capped_score(dot[i] * row_scale[i], mods.softcap);
        if (penalised) s -= distance_penalty(pen_w[i], pen_r[i], pos[i] - j);
      }
      const float m_new = fmaxf(m[i], warp_max(s));
      float alpha = 1.f, p = 0.f;
      if (m_new != -CUDART_INF_F) {                        // else: nothing seen yet, nothing to rescale
        alpha = expf(m[i] - m_new);
        p = valid ? expf(s - m_new) : 0.f;
      }
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < VPL; ++c) acc[i][c] *= alpha;
      p_s[(warp * kRowsPerWarp + i) * kKeys + lane] = p;
    }
    __syncwarp();
    const int n_here = min(kKeys, last_key - jb + 1);
    for (int jj = 0; jj < n_here; ++jj) {
      float pj[kRowsPerWarp];
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) pj[i] = p_s[(warp * kRowsPerWarp + i) * kKeys + jj];
      const float* vr = v_s + jj * vs;
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int col = lane + 32 * c;
        const float v = col < dv ? vr[col] : 0.f;
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) acc[i][c] += pj[i] * v;
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int row = r0 + warp * kRowsPerWarp + i;
    if (row >= rows) continue;
    if (sliced) {
      const size_t slab = (((size_t)e * nkv + kvh) * nsplit + blockIdx.x) * kRows + (row - r0);
#pragma unroll
      for (int c = 0; c < VPL; ++c) {
        const int col = lane + 32 * c;
        if (col < dv) part_o[slab * dv + col] = acc[i][c];
      }
      if (lane == 0) {
        part_ml[slab * 2] = m[i];
        part_ml[slab * 2 + 1] = l[i];
      }
      continue;
    }
    const float inv = head_gate_of(gate, (size_t)(t0 + row / G), kvh * G + row % G) / l[i];
    TO* o = out + ((size_t)(t0 + row / G) * nq + kvh * G + row % G) * dv;
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int col = lane + 32 * c;
      if (col < dv) o[col] = from_float<TO>(acc[i][c] * inv);
    }
  }
}

// One block per (entry, KV head, row): adds the slices' sums in slice order.  rows_padded: rows a slice holds
// per (entry, KV head) in part_o / part_ml (a multiple of 16).  Each slice's weight exp(m_s - M) is formed once.
constexpr int kMaxSlices = 64;

template <typename TO>
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       TO* __restrict__ out, const int* __restrict__ cu_q, int n_entries, int nq,
                                       int nkv, int dv, int nsplit, int rows_padded, HeadGate gate) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  __shared__ float w[kMaxSlices];
  __shared__ float inv_l;
  const long long b = blockIdx.x;
  const int r = (int)(b % rows_padded), kvh = (int)((b / rows_padded) % nkv), e = (int)(b / ((long long)rows_padded * nkv));
  const int G = nq / nkv, t0 = cu_q[e], rows = (cu_q[e + 1] - t0) * G;
  if (r >= rows) return;
  const size_t first = (((size_t)e * nkv + kvh) * nsplit) * rows_padded + r;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float M = -CUDART_INF_F;
    for (int s = lane; s < nsplit; s += 32) M = fmaxf(M, part_ml[(first + (size_t)s * rows_padded) * 2]);
    M = warp_max(M);
    float L = 0.f;
    for (int s = lane; s < nsplit; s += 32) {
      const float ms = part_ml[(first + (size_t)s * rows_padded) * 2];
      const float ws = ms != -CUDART_INF_F ? expf(ms - M) : 0.f;
      w[s] = ws;
      L += part_ml[(first + (size_t)s * rows_padded) * 2 + 1] * ws;
    }
    L = warp_sum(L);
    if (lane == 0) inv_l = head_gate_of(gate, (size_t)(t0 + r / G), kvh * G + r % G) / L;
  }
  __syncthreads();
  TO* o = out + ((size_t)(t0 + r / G) * nq + kvh * G + r % G) * dv;
  for (int col = threadIdx.x; col < dv; col += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < nsplit; ++s) a += part_o[(first + (size_t)s * rows_padded) * dv + col] * w[s];
    o[col] = from_float<TO>(a * inv_l);
  }
}

// One block per token: q = projection + bias into its own buffer (float32 or bfloat16); k and v = projection +
// bias; with a rotation table (cos, sin float32 [T, pairs]) the first 2 * pairs elements of every q and k head are
// turned behind the bias, pair i by the token's angle i: the partners are the elements (i, i + pairs), or (2i, 2i + 1)
// when interleaved, and (u, v) becomes (u cos - v sin, v cos + u sin); the rest of a head passes unchanged.
// mix_mode 1 keeps v (float32, [T, nkv * dv]) for later layers, mix_mode 2 replaces v by
// (1 - lambda) v + lambda kept; k and the final v go to the pages (kv_slot[t] = page * page_size + offset).
// write_kv 0 with mix_mode 0: the projection holds the q columns only.
template <typename TP>
__device__ __forceinline__ float rotated_element(const TP* __restrict__ x, const float* __restrict__ b, int d,
                                                 const float* __restrict__ cs, const float* __restrict__ sn, int pairs,
                                                 int interleaved) {
  // x, b: the head's elements and biases (b may be null); d: the element wanted
  const float own = to_float(x[d]) + (b ? b[d] : 0.f);
  if (d >= 2 * pairs) return own;
  int i, partner;
  bool first;
  if (interleaved) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
  else { first = d < pairs; i = first ? d : d - pairs; partner = first ? d + pairs : d - pairs; }
  const float other = to_float(x[partner]) + (b ? b[partner] : 0.f);
  const float c = cs[i], sgn = sn[i];
  return first ? own * c - other * sgn : own * c + other * sgn;
}

template <typename TP, typename TC>
__global__ void attention_bias_append_kernel(const TP* __restrict__ proj, long long ldp, const float* __restrict__ bias,
                                             float* __restrict__ q_out, bf16* __restrict__ q_out_bf16,
                                             TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                             const int* __restrict__ kv_slot,
                                             float* __restrict__ v_keep, const float* __restrict__ lambda,
                                             int mix_mode, int write_kv, int nq, int nkv, int dk, int dv,
                                             int page_size, const float* __restrict__ cos_t,
                                             const float* __restrict__ sin_t, int pairs, int interleaved) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const int t = blockIdx.x;
  const TP* p = proj + (size_t)t * ldp;
  const int nqd = nq * dk, nkd = nkv * dk, nvd = nkv * dv;
  const float* cs = pairs ? cos_t + (size_t)t * pairs : nullptr;
  const float* sn = pairs ? sin_t + (size_t)t * pairs : nullptr;
  for (int c = threadIdx.x; c < nqd; c += blockDim.x) {
    const int h = c / dk, d = c - h * dk;
    const float v = rotated_element(p + (size_t)h * dk, bias ? bias + (size_t)h * dk : nullptr, d, cs, sn, pairs, interleaved);
    if (q_out_bf16) q_out_bf16[(size_t)t * nqd + c] = __float2bfloat16_rn(v);     // for kernels that take bfloat16 queries
    else q_out[(size_t)t * nqd + c] = v;
  }
  if (!write_kv && mix_mode == 0) return;
  const int slot = kv_slot[t];
  const size_t page = slot / page_size, off = slot % page_size;
  if (write_kv) {
    for (int c = threadIdx.x; c < nkd; c += blockDim.x) {
      const int h = c / dk, d = c - h * dk;
      const float v = rotated_element(p + nqd + (size_t)h * dk, bias ? bias + nqd + (size_t)h * dk : nullptr, d, cs, sn,
                                      pairs, interleaved);
      k_cache[((page * nkv + h) * page_size + off) * dk + d] = from_float<TC>(v);
    }
  }
  const float lam = mix_mode == 2 ? lambda[0] : 0.f;
  for (int c = threadIdx.x; c < nvd; c += blockDim.x) {
    const int h = c / dv, d = c - h * dv;
    float v = to_float(p[nqd + nkd + c]) + (bias ? bias[nqd + nkd + c] : 0.f);
    if (mix_mode == 1) v_keep[(size_t)t * nvd + c] = v;
    if (mix_mode == 2) v = (1.f - lam) * v + lam * v_keep[(size_t)t * nvd + c];
    if (write_kv) v_cache[((page * nkv + h) * page_size + off) * dv + d] = from_float<TC>(v);
  }
}

// One block per token: every q head and every k head of a stacked q | k | v projection is divided by
// its root mean square, sqrt(mean(x^2) + eps), in float32 (eps <= 0: left as projected); q goes to its
// own buffer (float32, or bfloat16 for the kernels that take their queries so), k and v to the pages.
// A warp takes a head at a time and adds the squares in an order fixed by the head size.
template <typename TP, typename TC>
__global__ void attention_unit_norm_append_kernel(const TP* __restrict__ proj, long long ldp, float eps,
                                                  float* __restrict__ q_out, bf16* __restrict__ q_out_bf16,
                                                  TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                                  const int* __restrict__ kv_slot, int write_kv, int nq, int nkv,
                                                  int dk, int dv, int page_size) {
  pdl_wait();        // launched as a dependent of the kernel ahead: nothing is read before it has finished
  pdl_trigger();
  const int t = blockIdx.x;
  const TP* p = proj + (size_t)t * ldp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int slot = kv_slot[t];
  const size_t page = slot / page_size, off = slot % page_size;
  for (int h = warp; h < nq + nkv; h += warps) {
    const bool is_q = h < nq;
    if (!is_q && !write_kv) continue;
    const TP* x = p + (size_t)h * dk;                       // the k heads follow the q heads, all dk wide
    float inv = 1.f;
    if (eps > 0.f) {
      float ss = 0.f;
      for (int d = lane; d < dk; d += 32) {
        const float v = to_float(x[d]);
        ss += v * v;
      }
      inv = 1.f / sqrtf(warp_sum(ss) / (float)dk + eps);
    }
    for (int d = lane; d < dk; d += 32) {
      const float v = to_float(x[d]) * inv;
      if (is_q) {
        if (q_out_bf16) q_out_bf16[((size_t)t * nq + h) * dk + d] = __float2bfloat16_rn(v);
        else q_out[((size_t)t * nq + h) * dk + d] = v;
      } else {
        k_cache[((page * nkv + (h - nq)) * page_size + off) * dk + d] = from_float<TC>(v);
      }
    }
  }
  if (write_kv) {
    const TP* v_in = p + (size_t)(nq + nkv) * dk;
    for (int c = threadIdx.x; c < nkv * dv; c += blockDim.x) {
      const int h = c / dv, d = c - h * dv;
      v_cache[((page * nkv + h) * page_size + off) * dv + d] = from_float<TC>(to_float(v_in[c]));
    }
  }
}

template <typename TC, typename TO>
static int launch_general(int vpl, dim3 grid, size_t smem, cudaStream_t stream, const float* q, const void* k_cache,
                          const void* v_cache, void* out, const int* block_table, int table_stride, const int* cu_q,
                          const int* kv_lens, const float* sinks, int nq, int nkv, int dk, int dv, int page_size,
                          float scale, int window, int nsplit, int kv_chunk, float* part_o, float* part_ml,
                          int n_entries, ScoreMods mods, HeadGate gate) {
#define SRLM_GENERAL_CASE(V)                                                                                   \
  case V: {                                                                                                    \
    auto kern = paged_attention_general_kernel<TC, TO, V>;                                                     \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    launch_pdl(kern, dim3(grid), dim3(kWarps * 32), smem, stream, q, (const TC*)k_cache, (const TC*)v_cache, (TO*)out, block_table, \
                                              table_stride, cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size,  \
                                              scale, window, nsplit, kv_chunk, part_o, part_ml, mods, gate);   \
    break;                                                                                                     \
  }
  switch (vpl) {
    SRLM_GENERAL_CASE(1)
    SRLM_GENERAL_CASE(2)
    SRLM_GENERAL_CASE(4)
    SRLM_GENERAL_CASE(8)
    SRLM_GENERAL_CASE(16)
  }
#undef SRLM_GENERAL_CASE
  if (nsplit > 1) {
    const long long blocks = (long long)n_entries * nkv * kRows;
    launch_pdl(attention_merge_kernel<TO>, dim3((unsigned)blocks), dim3(128), 0, stream, part_o, part_ml, (TO*)out, cu_q, n_entries, nq,
                                                                     nkv, dv, nsplit, kRows, gate);
  }
  return launched();
}

}  // namespace srlm

using namespace srlm;

// q: float32 [T, nq, dk]; k_cache [pages, nkv, page_size, dk]; v_cache [pages, nkv, page_size, dv] or
// null (the values are the keys' first dv elements); out [T, nq, dv] in out_dtype; sinks: float32 [nq] or null.
extern "C" int srlm_paged_attention_general(const float* q, const void* k_cache, const void* v_cache, void* out,
                                            int cache_dtype, int out_dtype, const int* block_table,
                                            int table_stride, const int* cu_q, const int* kv_lens,
                                            const float* sinks, int n_entries, int max_q_len, int nq, int nkv,
                                            int dk, int dv, int page_size, float scale, int window, int nsplit,
                                            int kv_chunk, float* part_o, float* part_ml, const float* head_scale,
                                            const float* pen_weight, const float* pen_rate, float softcap,
                                            const float* gate_logits, long long ld_gate, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return ST_OK;
  const HeadGate gate{gate_logits, ld_gate};
  if ((pen_weight == nullptr) != (pen_rate == nullptr))
    return refuse(ST_BAD_SIZE, "paged_attention_general: a distance penalty needs its weight and its rate");
  const ScoreMods mods{head_scale, pen_weight, pen_rate, softcap};
  if (nq <= 0 || nkv <= 0 || nq % nkv || dk <= 0 || dv <= 0 || dv > 512 || page_size <= 0 || (!v_cache && dv > dk))
    return refuse(ST_BAD_SIZE, "paged_attention_general: nq=%d nkv=%d dk=%d dv=%d page_size=%d (dv <= 512; values "
                  "read from the keys need dv <= dk)", nq, nkv, dk, dv, page_size);
  if (n_entries > 65535 || nkv > 65535) return refuse(ST_BAD_SIZE, "paged_attention_general: %d entries", n_entries);
  const size_t smem = ((size_t)kRows * dk + (size_t)kKeys * (dk + 1) + (v_cache ? (size_t)kKeys * dv : 0) +
                       (size_t)kRows * kKeys) * sizeof(float);
  if (smem > 220 * 1024) return refuse(ST_BAD_SIZE, "paged_attention_general: dk=%d dv=%d need %zu bytes of shared memory", dk, dv, smem);
  const int G = nq / nkv;
  const long long tiles = ((long long)max_q_len * G + kRows - 1) / kRows;
  if (nsplit > 1 && (tiles != 1 || kv_chunk <= 0 || kv_chunk % kKeys || !part_o || !part_ml))
    return refuse(ST_BAD_SIZE, "paged_attention_general: %d slices of %d keys need entries of at most %d rows, slices "
                  "of whole key blocks and a workspace", nsplit, kv_chunk, kRows);
  if (nsplit > kMaxSlices) return refuse(ST_BAD_SIZE, "paged_attention_general: at most %d slices", kMaxSlices);
  if (nsplit < 1) nsplit = 1;
  dim3 grid((unsigned)(nsplit > 1 ? nsplit : tiles), (unsigned)nkv, (unsigned)n_entries);
  int vpl = 1;
  while (vpl * 32 < dv) vpl <<= 1;
  if (cache_dtype == DT_F32 && out_dtype == DT_F32)
    return launch_general<float, float>(vpl, grid, smem, stream, q, k_cache, v_cache, out, block_table, table_stride,
                                        cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size, scale, window, nsplit, kv_chunk,
                                        part_o, part_ml, n_entries, mods, gate);
  if (cache_dtype == DT_BF16 && out_dtype == DT_F32)
    return launch_general<bf16, float>(vpl, grid, smem, stream, q, k_cache, v_cache, out, block_table, table_stride,
                                       cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size, scale, window, nsplit, kv_chunk,
                                        part_o, part_ml, n_entries, mods, gate);
  if (cache_dtype == DT_BF16 && out_dtype == DT_BF16)
    return launch_general<bf16, bf16>(vpl, grid, smem, stream, q, k_cache, v_cache, out, block_table, table_stride,
                                      cu_q, kv_lens, sinks, nq, nkv, dk, dv, page_size, scale, window, nsplit, kv_chunk,
                                        part_o, part_ml, n_entries, mods, gate);
  return refuse(ST_BAD_DTYPE, "paged_attention_general: cache dtype %d with output dtype %d", cache_dtype, out_dtype);
}

// proj: [T, ldp] in proj_dtype, columns q (nq * dk), k (nkv * dk), v (nkv * dv); bias: float32 over the
// same columns or null.  mix_mode 0: v as it is; 1: also kept in v_keep; 2: mixed with v_keep by lambda[0].
// cos_t, sin_t float32 [T, pairs] (pairs 0: no rotation): q and k heads turned behind the bias, see the kernel.
extern "C" int srlm_attention_bias_append(const void* proj, int proj_dtype, long long ldp, const float* bias,
                                          void* q_out, int q_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                          const int* kv_slot, float* v_keep, const float* lambda, int mix_mode,
                                          int write_kv, int T, int nq, int nkv, int dk, int dv, int page_size,
                                          const float* cos_t, const float* sin_t, int pairs, int interleaved,
                                          cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  const bool q_only = !write_kv && mix_mode == 0;
  if (nq <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 ||
      ldp < (long long)nq * dk + (q_only ? 0 : (long long)nkv * (dk + dv)) ||
      (mix_mode != 0 && !v_keep) || (mix_mode == 2 && !lambda) || mix_mode < 0 || mix_mode > 2)
    return refuse(ST_BAD_SIZE, "attention_bias_append: nq=%d nkv=%d dk=%d dv=%d ldp=%lld mix_mode=%d", nq, nkv, dk, dv,
                  ldp, mix_mode);
  if (pairs < 0 || 2 * pairs > dk || (pairs > 0 && (!cos_t || !sin_t)))
    return refuse(ST_BAD_SIZE, "attention_bias_append: %d rotated pairs in heads of %d need their tables", pairs, dk);
#define SRLM_APPEND(TP, TC)                                                                                       \
  launch_pdl(attention_bias_append_kernel<TP, TC>, dim3(T), dim3(256), 0, stream, (const TP*)proj, ldp, bias, q_dtype == DT_F32 ? (float*)q_out : nullptr, q_dtype == DT_BF16 ? (bf16*)q_out : nullptr, (TC*)k_cache,    \
                                                              (TC*)v_cache, kv_slot, v_keep, lambda, mix_mode,   \
                                                              write_kv, nq, nkv, dk, dv, page_size, cos_t, sin_t, pairs, interleaved)
  if (proj_dtype == DT_F32 && cache_dtype == DT_F32) SRLM_APPEND(float, float);
  else if (proj_dtype == DT_F32 && cache_dtype == DT_BF16) SRLM_APPEND(float, bf16);
  else if (proj_dtype == DT_BF16 && cache_dtype == DT_BF16) SRLM_APPEND(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "attention_bias_append: projection dtype %d with cache dtype %d", proj_dtype, cache_dtype);
#undef SRLM_APPEND
  return launched();
}

// Adds the slices that a sliced attention kernel left in part_o [.., rows_padded, dv] / part_ml [.., rows_padded, 2].
extern "C" int srlm_attention_general_merge(const float* part_o, const float* part_ml, void* out, int out_dtype,
                                            const int* cu_q, int n_entries, int nq, int nkv, int dv, int nsplit,
                                            int rows_padded, const float* gate_logits, long long ld_gate,
                                            cudaStream_t stream) {
  if (n_entries <= 0 || nsplit <= 1) return ST_OK;
  const HeadGate gate{gate_logits, ld_gate};
  if (nsplit > kMaxSlices || rows_padded <= 0)
    return refuse(ST_BAD_SIZE, "attention_general_merge: %d slices (at most %d), %d rows", nsplit, kMaxSlices, rows_padded);
  const long long blocks = (long long)n_entries * nkv * rows_padded;
  if (out_dtype == DT_F32)
    launch_pdl(attention_merge_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, part_o, part_ml, (float*)out, cu_q, n_entries, nq,
                                                                        nkv, dv, nsplit, rows_padded, gate);
  else if (out_dtype == DT_BF16)
    launch_pdl(attention_merge_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, part_o, part_ml, (bf16*)out, cu_q, n_entries, nq,
                                                                       nkv, dv, nsplit, rows_padded, gate);
  else
    return refuse(ST_BAD_DTYPE, "attention_general_merge: output dtype %d", out_dtype);
  return launched();
}

// proj: [T, ldp] in proj_dtype, columns q (nq * dk), k (nkv * dk), v (nkv * dv), then whatever else the
// projection carries.  q and k heads divided by sqrt(mean(x^2) + eps) (eps <= 0: not), q to q_out, k and v to the pages.
extern "C" int srlm_attention_unit_norm_append(const void* proj, int proj_dtype, long long ldp, float eps, void* q_out,
                                               int q_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                               const int* kv_slot, int write_kv, int T, int nq, int nkv, int dk, int dv,
                                               int page_size, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (nq <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || ldp < (long long)nq * dk + (long long)nkv * (dk + dv))
    return refuse(ST_BAD_SIZE, "attention_unit_norm_append: nq=%d nkv=%d dk=%d dv=%d ldp=%lld", nq, nkv, dk, dv, ldp);
#define SRLM_APPEND(TP, TC)                                                                                       \
  launch_pdl(attention_unit_norm_append_kernel<TP, TC>, dim3(T), dim3(256), 0, stream, (const TP*)proj, ldp, eps, \
             q_dtype == DT_F32 ? (float*)q_out : nullptr, q_dtype == DT_BF16 ? (bf16*)q_out : nullptr,            \
             (TC*)k_cache, (TC*)v_cache, kv_slot, write_kv, nq, nkv, dk, dv, page_size)
  if (proj_dtype == DT_F32 && cache_dtype == DT_F32) SRLM_APPEND(float, float);
  else if (proj_dtype == DT_F32 && cache_dtype == DT_BF16) SRLM_APPEND(float, bf16);
  else if (proj_dtype == DT_BF16 && cache_dtype == DT_BF16) SRLM_APPEND(bf16, bf16);
  else return refuse(ST_BAD_DTYPE, "attention_unit_norm_append: projection dtype %d with cache dtype %d", proj_dtype, cache_dtype);
#undef SRLM_APPEND
  return launched();
}
