"""Loads ``libsrlm_kernels.so`` and wraps each exported kernel for torch tensors.

There is no other implementation behind these functions: if the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
Tensors are passed as raw device pointers; every launch goes to torch's
current stream, so the calls can be recorded into a CUDA graph.
"""
from __future__ import annotations

import ctypes as C
import functools
from typing import Optional

import torch

from ..errors import ShapeError, Unavailable

DT_F32, DT_BF16 = 0, 1
_CODES = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _CODES[dt]
    except KeyError:
        raise ShapeError(f"dtype {dt} is not taken by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return C.c_void_p(0)
    if not t.is_cuda:
        raise Unavailable("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise ShapeError("kernels take contiguous tensors")
    return C.c_void_p(t.data_ptr())


# torch.cuda.current_stream() builds a Stream object through several Python layers (3.4 us measured, a
# third of a launch's host cost); the two calls below are what it ends in.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_CURRENT_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current CUDA stream of the current device (the capturing one while a graph is recorded)."""
    if _RAW_STREAM is not None and _CURRENT_DEVICE is not None:
        return C.c_void_p(_RAW_STREAM(_CURRENT_DEVICE()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class KernelLibrary:
    def __init__(self):
        self._lib = None
        self.launches = 0          # kernels launched through this object (a benchmark reports it)
        self.force_simt_gemm = False   # tests: run the float32 FMA twin in place of the tensor cores
        self.force_simt_attention = False
        self.force_tcgen05_gemm = False
        # The weight-streaming (mma.sync) kernel serves products of at most this many tokens and weight rows.
        # 0: none -- the one-tile tensor-core kernel with its K splits in a cluster streams the weights faster
        # at every token count (a layer's four products at 8 tokens: 70.8 against 82.8 us); 8 brings it back.
        self.skinny_max_tokens = 0
        self.skinny_max_rows = 1 << 30
        self.force_cp_async_decode = False
        self.cluster_decode_merge = True        # slices of decode attention merged in a thread-block cluster
        self.fuse_decode_attention = True       # decode: norm, rotation and append inside the attention kernel
        self.force_mma_sync_prefill = False
        self.split_mixed_attention = True       # mixed steps: decoding requests to the keys-split kernel ...
        self.split_prefill_keys = True          # rows-split attention: the keys in slices when rows are few
        self.split_mixed_min_blocks = None      # ... when they make this many blocks (None: one per SM)
        self.fuse_norms_into_products = True    # steps of up to 128 tokens: the blocks' norms inside the products
        self.early_launch = True                # weight-streaming products may start under the kernel ahead of them
        self.split_general_attention = True     # decode steps of the general attention: the keys in slices
        self.general_attention_on_tensor_cores = True   # its prompts and portions: mma.sync, when the sizes fit
        self.latent_prompts_in_head_space = True        # latent attention: prompts form per-head keys and values
        self.sinks_in_tcgen05_prefill = True            # attention with sinks, heads of 128: prompts on the tcgen05 kernel
        self.grouped_products_on_tensor_cores = True    # routed experts in bfloat16: mma.sync, when the sizes fit
        self.grouped_products_in_tensor_memory = True   # ... and steps of many tokens: the persistent tcgen05 kernel
        self.grouped_pairs = True                       # ... whose largest steps run pairs of SMs on tiles of 256 tokens

    @property
    def lib(self):
        if self._lib is None:
            from ..csrc.build import build_kernels
            try:
                path = build_kernels()
                self._lib = C.CDLL(path)
            except Exception as e:   # noqa: BLE001
                raise Unavailable(f"the CUDA kernel library is missing and could not be built: {e}") from e
            self._lib.srlm_last_error.restype = C.c_char_p
            import os
            if os.environ.get("SRLM_PDL", "1") == "0":     # plain stream order between kernels
                self._lib.srlm_set_pdl(0)
        return self._lib

    def sm_count(self, device) -> int:
        counts = self.__dict__.setdefault("_sm_counts", {})
        if device not in counts:
            counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
        return counts[device]

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch between the kernels of a step (on by default)."""
        self.lib.srlm_set_pdl(C.c_int(1 if on else 0))

    def begin_timing(self) -> None:
        """From now on every launch is followed by a CUDA event; ``end_timing`` turns the gaps between
        consecutive events into a table.  Kernels of one stream run one after the other, so the gap
        before a launch's event is that kernel's time (with its launch gap; no overlap between kernels
        is possible while this is on: use it on eager steps, for shares, not for absolutes; launches that
        go into a CUDA graph under capture are left out)."""
        start = torch.cuda.Event(enable_timing=True)
        start.record()
        self._timing = [("", start)]

    def end_timing(self) -> dict:
        """{kernel name: (launches, milliseconds)} since begin_timing (waits for the device)."""
        marks, self._timing = getattr(self, "_timing", None) or [], None
        torch.cuda.synchronize()
        table: dict = {}
        for (_, before), (name, after) in zip(marks, marks[1:]):
            n, ms = table.get(name, (0, 0.0))
            table[name] = (n + 1, ms + before.elapsed_time(after))
        return table

    def _check(self, status: int, what: str):
        self.launches += 1
        if getattr(self, "_timing", None) is not None and status == 0 \
                and not torch.cuda.is_current_stream_capturing():      # a timed event cannot be recorded into a graph
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._timing.append((what, ev))
        if status != 0:
            msg = self.lib.srlm_last_error().decode(errors="replace")
            if status < 0:
                raise ShapeError(f"{what} refused: {msg}")
            raise RuntimeError(f"{what} failed with CUDA error {status}: {msg}")

    # ---- elementwise -----------------------------------------------------
    def embed_gather(self, ids, table, out, bad_flag):
        T, H = out.shape
        self._check(self.lib.srlm_embed_gather(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out),
                                               C.c_int(T), C.c_int(H), C.c_int(table.shape[0]),
                                               _ptr(bad_flag), _stream()), "embed_gather")

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None, unit_offset=False):
        R, H = out.shape
        self._check(self.lib.srlm_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), C.c_float(eps),
                                              _ptr(out), dtype_code(out.dtype), _ptr(rows), C.c_int(R),
                                              C.c_int(H), C.c_int(int(unit_offset)), _stream()),
                    "add_rmsnorm")

    def swiglu(self, gate_up, out):
        T, I = out.shape
        self._check(self.lib.srlm_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), C.c_int(T),
                                         C.c_int(I), _stream()), "swiglu")

    def cast(self, src, dst):
        self._check(self.lib.srlm_cast(_ptr(src), dtype_code(src.dtype), _ptr(dst), dtype_code(dst.dtype),
                                       C.c_longlong(src.numel()), _stream()), "cast")

    def cast_columns(self, src, column, dst):
        """dst [T, width] (contiguous, float32 or bfloat16) = the float32 columns [column, column + width) of src."""
        T, width = dst.shape
        if src.dtype != torch.float32 or src.stride(1) != 1 or src.shape[1] < column + width or src.shape[0] != T:
            raise ShapeError("cast_columns: float32 columns of a row-major tensor")
        self._check(self.lib.srlm_cast_columns(C.c_void_p(src.data_ptr() + 4 * column), C.c_longlong(src.stride(0)),
                                               _ptr(dst), dtype_code(dst.dtype), C.c_int(T), C.c_int(width), _stream()),
                    "cast_columns")

    def patch_words(self, words, pairs, src, n, flag):
        """words[pairs[2 i]] = src[pairs[2 i + 1]] for i < n, all int32 on the device: token ids that a step
        takes from what the step before it sampled, before the host has read them.  An index outside its
        tensor is skipped and raises flag[0]."""
        if any(t.dtype != torch.int32 for t in (words, pairs, src, flag)) or pairs.numel() < 2 * n:
            raise ShapeError("patch_words: int32 tensors, two words a pair")
        self._check(self.lib.srlm_patch_words(_ptr(words), C.c_longlong(words.numel()), _ptr(pairs), _ptr(src),
                                              C.c_int(src.numel()), C.c_int(n), _ptr(flag), _stream()), "patch_words")

    def check_finite(self, a, b, flag):
        """flag[0] = 1 if any element of a (+ b, same shape, when given) is NaN or infinite; a float32."""
        if a.dtype != torch.float32 or (b is not None and b.numel() != a.numel()):
            raise ShapeError("check_finite: a must be float32 and b of the same size")
        self._check(self.lib.srlm_check_finite(_ptr(a), _ptr(b), dtype_code(b.dtype) if b is not None else DT_F32,
                                               C.c_longlong(a.numel()), _ptr(flag), _stream()), "check_finite")

    def residual_add(self, residual, delta):
        self._check(self.lib.srlm_residual_add(_ptr(residual), _ptr(delta), dtype_code(delta.dtype),
                                               C.c_longlong(delta.numel()), _stream()), "residual_add")

    # ---- position encoding and cache append ------------------------------
    def rope_table(self, positions, cos, sin, theta, rotary_dim):
        T, half = cos.shape
        self._check(self.lib.srlm_rope_table(_ptr(positions), _ptr(cos), _ptr(sin), C.c_int(T), C.c_int(half),
                                             C.c_double(theta), C.c_int(rotary_dim), _stream()), "rope_table")

    def rope_table_freq(self, positions, freq, cos, sin, length=1.0):
        """cos / sin [T, half] of position * freq[i], times ``length``; freq float64 [half] on the device."""
        T, half = cos.shape
        if freq.dtype != torch.float64 or freq.numel() != half:
            raise ShapeError("rope_table_freq: one float64 frequency per pair")
        self._check(self.lib.srlm_rope_table_freq(_ptr(positions), _ptr(freq), _ptr(cos), _ptr(sin), C.c_int(T),
                                                  C.c_int(half), C.c_double(length), _stream()), "rope_table_freq")

    def qk_norm_rope_append(self, qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, eps, cos, sin, kv_slot,
                            nq, nkv, hd, rotary_half, write_kv=True, interleaved=False):
        """k_cache / v_cache: [pages, kv_heads, page_size, head_dim]; kv_slot[t] = page * page_size + offset.
        cos / sin [T, rotary_half] rotate the pairs (i, i + rotary_half), or (2i, 2i + 1) when interleaved,
        of the first 2 * rotary_half elements of every q and k head; rotary_half 0: no rotation."""
        T = qkv.shape[0]
        self._check(self.lib.srlm_qk_norm_rope_append(
            _ptr(qkv), _ptr(q_out), dtype_code(qkv.dtype), _ptr(k_cache), _ptr(v_cache),
            dtype_code(k_cache.dtype), _ptr(q_norm_w), _ptr(k_norm_w), C.c_float(eps), _ptr(cos), _ptr(sin),
            _ptr(kv_slot), C.c_int(T), C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(rotary_half),
            C.c_int(int(write_kv)), C.c_int(k_cache.shape[2]), C.c_int(int(interleaved)), _stream()),
            "qk_norm_rope_append")

    # ---- attention --------------------------------------------------------
    def paged_attention_simt(self, q, k_cache, v_cache, out, block_table, entry_of_token, positions,
                             nq, nkv, hd, page_size, scale, window=0):
        T = q.shape[0]
        self._check(self.lib.srlm_paged_attention_simt(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), dtype_code(q.dtype), dtype_code(k_cache.dtype),
            _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(entry_of_token), _ptr(positions),
            C.c_int(T), C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale),
            C.c_int(window or 0), _stream()), "paged_attention_simt")

    # ---- matrix products ----------------------------------------------------
    def gemm_tn_simt(self, a, w, out):
        """out[M,N] = a[M,K] @ w[N,K]^T, float32 FMA accumulation."""
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise ShapeError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.srlm_gemm_tn_simt(
            _ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype),
            C.c_int(M), C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0)), _stream()), "gemm_tn_simt")

    # split-K workspace of the tensor-core GEMM: 64 KiB of tile counters, then float32 partials
    GEMM_WS_BYTES = 65536 + (64 << 20)

    def _gemm_state(self, device):
        st = getattr(self, "_gemm_ws", None)
        if st is None or st[0].device != device:
            ws = torch.zeros(self.GEMM_WS_BYTES, dtype=torch.uint8, device=device)
            err = torch.zeros(1, dtype=torch.int32, device=device)
            st = self._gemm_ws = (ws, err)
        bound = getattr(self, "_bound_err", None)
        if bound is not None and bound.device == device:
            return st[0], bound
        return st

    def bind_error_flag(self, flag: Optional[torch.Tensor]) -> None:
        """The int32 word that kernels with bounded waits (TMA / tensor-core pipelines) raise when a wait
        runs out.  An engine binds a word of its own status buffer before each forward, so that the
        step's read-back sees it; None goes back to the library's own word."""
        self._bound_err = flag

    def wait_probe(self, flag: torch.Tensor, limit_cycles: int = 1_000_000, code: int = 99) -> None:
        """A kernel whose one bounded wait (the pipelines' own, on a barrier nobody arrives at) runs out after
        ``limit_cycles`` and writes ``code`` to flag[0], then ends normally.  For tests of the way from such a
        wait to the host; the product path never launches it."""
        if flag.dtype != torch.int32:
            raise ShapeError("wait_probe: an int32 flag")
        self._check(self.lib.srlm_wait_probe(_ptr(flag), C.c_longlong(limit_cycles), C.c_int(code), _stream()),
                    "wait_probe")

    def gemm_error_flag(self, device) -> int:
        """Nonzero if a kernel gave up on a bounded wait since the flag was last read (synchronises)."""
        err = self._gemm_state(device)[1]
        v = int(err.item())
        if v:
            err.zero_()
        return v

    # The plans below are made on the host, also where there is no GPU (tests).  They are tuned for the
    # B200's 148 SMs, and the token-tile rule repeats the one in gemm_tcgen05.cu
    # (srlm_gemm_tcgen05_token_tile reports the kernel's own choice; a GPU test holds the two together).
    SMS = 148
    BN256_MIN_TILES = 96

    @staticmethod
    @functools.lru_cache(maxsize=4096)
    def gemm_token_tile(M: int, N: int) -> int:
        """The width of the token tiles of the tensor-core product of M tokens and N weight rows (the rule
        of token_tile in gemm_tcgen05.cu, where its reasons and measurements stand)."""
        if M <= 128:
            return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        rows128 = (N + 127) // 128
        if rows128 * ((M + 255) // 256) >= KernelLibrary.BN256_MIN_TILES:
            return 256
        sms = KernelLibrary.SMS
        tiles128, tiles256 = rows128 * ((M + 127) // 128), ((N + 255) // 256) * ((M + 255) // 256)
        rounds128, rounds256 = -(-tiles128 // sms), -(-tiles256 // (sms // 2))
        return 256 if 4 * rounds256 < 3 * rounds128 else 128

    @staticmethod
    @functools.lru_cache(maxsize=4096)
    def gemm_splits(M: int, N: int, K: int) -> int:
        """How many ways to split K: the number of blocks should fill whole waves of the SMs
        (192 tiles alone would leave the second wave two thirds empty), each split keeping at
        least 4 k-blocks, the partial sums fitting the workspace."""
        bn = KernelLibrary.gemm_token_tile(M, N)
        if bn == 256:
            return 1                      # pairs of SMs on whole tiles of 256 x 256
        tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
        total_kb = (K + 63) // 64
        if tiles >= 1024:
            return 1
        if M > 16:
            # Measured on B200, 8B layer sizes: splitting until about 200 blocks stream (a few more up to 32
            # tokens) pays, each split keeping at least 8 k-blocks.  Up to 8 splits add their sums inside a
            # thread-block cluster; with that, 4 splits also pay from 65 to a few hundred tokens, where
            # an unsplit product of a narrow output leaves most SMs without a tile (128 tokens: o and down
            # projections 27.6 -> 21.5 us and 64.5 -> 35.6 us).
            if M <= 32:
                sp = min(222 // max(1, tiles), total_kb // 8)
            elif M <= 64:
                sp = min(200 // max(1, tiles), total_kb // 8, 8)
            else:
                # tiles of 128 tokens, two blocks to an SM: up to about 256 blocks run as one round (clusters
                # of 3 or 4 do not pack the GPCs to the last slot: 288 blocks measured a round more).  At 256
                # tokens, 14B sizes: down projection 61.5 -> 53.3 us with 3 splits instead of 2 (80 tiles),
                # 8B sizes: 36.1 -> 31.3 us with 4 instead of 3 (64 tiles); 512 tokens, 8B: 58.4 -> 51.8 us
                # with 2 splits of 128 tiles
                sp = min(256 // max(1, tiles), total_kb // 8, 4)
                if M <= 128:
                    # one token tile: a long K pays more splits (down projection of 128 tokens, 4096 x 12,288:
                    # 28.5 us in 4 splits, 25.6 in 6, 24.3 in 8; the output projection's K of 4096 does not)
                    sp = max(sp, min(256 // max(1, tiles), total_kb // 16, 8))
            sp = max(1, sp)
            if M <= 64 and sp == 1 and 148 < tiles and 2 * tiles <= 444 and total_kb >= 16:
                sp = 2        # three blocks of a shallower ring an SM (the kernel picks it by the block count)
            while sp > 8 and 65536 + sp * tiles * 128 * bn * 4 > KernelLibrary.GEMM_WS_BYTES:
                sp -= 1
            return sp
        # Up to 16 tokens three blocks share an SM (444 at a time); splits up to the cluster's 8.  Measured on
        # B200 at 16 tokens, 8B layer sizes (QKV / O / gate-up / down): 4-8 / 6-8 / 2 / 6-8 splits are best
        # (11.6 / 9.6 / 32.1 / 19.7 us; gate/up unsplit 35.0 us, in 3 splits 37.5 us; down in 9 splits through
        # the workspace 23.4 us).
        return max(1, min(444 // max(1, tiles), total_kb // 8, 8))

    def gemm_tn_tcgen05(self, a, w, out, splits=None, swiglu8=False):
        """out[M,N] = a[M,K] @ w[N,K]^T, bfloat16 operands, tcgen05 tensor cores, float32 accumulation.
        swiglu8: w's rows come in blocks of 16 (8 gate rows, then the 8 up rows of the same features)
        and out[M, N/2] = silu(gate) * up."""
        M, K = a.shape
        N = w.shape[0]
        if (w.shape[1] != K or tuple(out.shape) != (M, N // 2 if swiglu8 else N) or a.dtype != torch.bfloat16
                or w.dtype != torch.bfloat16):
            raise ShapeError(f"gemm_tcgen05: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, "
                             f"out {tuple(out.shape)}")
        ws, err = self._gemm_state(a.device)
        if splits is None:
            splits = self.gemm_splits(M, N, K)
        self._check(self.lib.srlm_gemm_tn_tcgen05(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), C.c_int(M), C.c_int(N), C.c_int(K),
            C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)), C.c_longlong(out.stride(0)), C.c_int(splits),
            _ptr(ws), C.c_longlong(ws.numel()), _ptr(err), C.c_int(int(swiglu8)), _stream()),
            f"gemm_tn_tcgen05[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None else "gemm_tn_tcgen05")

    FUSED_TOKENS = 128       # most tokens of a product that runs its norms inside itself

    def gemm_tn_tcgen05_fused(self, a, w, out=None, swiglu8=False, scale_parts=None, norm_width=0, eps=0.0,
                              residual=None, next_w=None, xw_out=None, ss_out=None):
        """The tensor-core product of at most 128 tokens fused with the norms around it: the same contract
        as gemm_tn_skinny_fused, except that the partial sums of squares lie as [parts, tokens]
        (scale_parts: any row stride; ss_out: [ceil(N / 128), >= M])."""
        M, K = a.shape
        N = w.shape[0]
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or M > self.FUSED_TOKENS:
            raise ShapeError(f"gemm_tcgen05_fused: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
        if residual is None and (out is None or tuple(out.shape) != (M, N // 2 if swiglu8 else N)):
            raise ShapeError("gemm_tcgen05_fused: out has the wrong shape")
        if ss_out is not None and (ss_out.shape[0] < (N + 127) // 128 or ss_out.shape[1] < M):
            raise ShapeError("gemm_tcgen05_fused: ss_out must be [ceil(N/128), >= M]")
        ws, err = self._gemm_state(a.device)
        self._check(self.lib.srlm_gemm_tn_tcgen05_fused(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else DT_BF16, C.c_int(M),
            C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0) if out is not None else N), C.c_int(self.gemm_splits(M, N, K)), _ptr(ws),
            C.c_longlong(ws.numel()), _ptr(err), C.c_int(int(swiglu8)), _ptr(scale_parts),
            C.c_int(scale_parts.shape[0] if scale_parts is not None else 0),
            C.c_longlong(scale_parts.stride(0) if scale_parts is not None else 0), C.c_int(norm_width), C.c_float(eps),
            _ptr(residual), C.c_longlong(residual.stride(0) if residual is not None else 0), _ptr(next_w),
            _ptr(xw_out), C.c_longlong(xw_out.stride(0) if xw_out is not None else 0), _ptr(ss_out),
            C.c_longlong(ss_out.stride(0) if ss_out is not None else 0), _stream()),
            f"gemm_tn_tcgen05_fused[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None
            else "gemm_tn_tcgen05_fused")

    def gemm_dealt_tiles(self, M: int, N: int, K: int) -> int:
        """How many tiles of this product the persistent tensor-core kernel deals out by k-blocks
        (0: whole tiles only, or another kernel serves these sizes)."""
        return int(self.lib.srlm_gemm_tcgen05_dealt_tiles(C.c_int(M), C.c_int(N), C.c_int(K)))

    def gemm_tn_skinny(self, a, w, out, swiglu8=False, early=True):
        """out[M,N] = a[M,K] @ w[N,K]^T for M <= 16: the weight-streaming kernel of decode steps.
        swiglu8: as in gemm_tn_tcgen05.  early: the kernel may start under the tail of the kernel ahead
        of it (it requests its first weights, then waits for that kernel's results); False for the
        product that follows a mixer's own kernel, where that measured much slower."""
        M, K = a.shape
        N = w.shape[0]
        if (w.shape[1] != K or tuple(out.shape) != (M, N // 2 if swiglu8 else N) or a.dtype != torch.bfloat16
                or w.dtype != torch.bfloat16):
            raise ShapeError(f"gemm_skinny: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, "
                             f"out {tuple(out.shape)}")
        self._check(self.lib.srlm_gemm_tn_skinny(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype), C.c_int(M), C.c_int(N), C.c_int(K),
            C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)), C.c_longlong(out.stride(0)),
            C.c_int(int(swiglu8)), C.c_int(int(early and self.early_launch)), _stream()),
            f"gemm_tn_skinny[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None else "gemm_tn_skinny")

    def gemm_tn_skinny_fused(self, a, w, out=None, swiglu8=False, scale_parts=None, norm_width=0, eps=0.0,
                             residual=None, next_w=None, xw_out=None, ss_out=None, early=True):
        """The weight-streaming product (at most 8 tokens) fused with the norms around it.

        scale_parts [parts, 8] float32: ``a`` holds bf16(residual * norm weight); the product is scaled per
        token by rsqrt(sum of the parts / norm_width + eps).  residual [M, N] float32: the product is added
        to it in place instead of being stored; with next_w [N] also xw_out[M, N] = bf16(residual * next_w)
        and ss_out [N/16, 8] (each block's share of the rows' sums of squares) are written."""
        M, K = a.shape
        N = w.shape[0]
        if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K or M > 8:
            raise ShapeError(f"gemm_skinny_fused: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}")
        if residual is None and (out is None or tuple(out.shape) != (M, N // 2 if swiglu8 else N)):
            raise ShapeError("gemm_skinny_fused: out has the wrong shape")
        if ss_out is not None and (ss_out.shape[0] < (N + 15) // 16 or ss_out.shape[1] != 8):
            raise ShapeError("gemm_skinny_fused: ss_out must be [ceil(N/16), 8]")
        self._check(self.lib.srlm_gemm_tn_skinny_fused(
            _ptr(a), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else DT_BF16, C.c_int(M),
            C.c_int(N), C.c_int(K), C.c_longlong(a.stride(0)), C.c_longlong(w.stride(0)),
            C.c_longlong(out.stride(0) if out is not None else N), C.c_int(int(swiglu8)), _ptr(scale_parts),
            C.c_int(scale_parts.shape[0] if scale_parts is not None else 0), C.c_int(norm_width), C.c_float(eps),
            _ptr(residual), C.c_longlong(residual.stride(0) if residual is not None else 0), _ptr(next_w),
            _ptr(xw_out), C.c_longlong(xw_out.stride(0) if xw_out is not None else 0), _ptr(ss_out),
            C.c_int(int(early and self.early_launch)), _stream()),
            f"gemm_tn_skinny_fused[{M}x{N}x{K}]" if getattr(self, "_timing", None) is not None
            else "gemm_tn_skinny_fused")

    def fuses_in_skinny(self, T: int, w) -> bool:
        """Whether a fused product of T tokens runs the weight-streaming kernel (else the tensor-core one)."""
        return T <= min(8, self.skinny_max_tokens) and w.shape[0] <= self.skinny_max_rows \
            and not self.force_tcgen05_gemm

    def can_fuse_norms(self, T: int, dtype, w) -> bool:
        """Whether a product of T tokens with this weight may run the norms around it inside itself: the
        weight-streaming kernel up to 8 tokens, the one-tile tensor-core kernel up to 128."""
        return (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T <= self.FUSED_TOKENS
                and w.shape[1] % 8 == 0 and not self.force_simt_gemm and self.fuse_norms_into_products)

    def can_fuse_swiglu(self, a_dtype, w) -> bool:
        """Whether gemm(..., swiglu8=True) is offered for these operands (the tensor-core kernels only)."""
        return (a_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
                and w.shape[0] % 16 == 0 and not self.force_simt_gemm)

    def gemm(self, a, w, out, swiglu8=False, early=True):
        """The product path's matrix product: picks the kernel for the dtypes and sizes.  bfloat16
        operands go to the tensor cores; float32 operands, and widths that TMA cannot address
        (K not a multiple of 8), go to the float32 FMA kernel.  early: see gemm_tn_skinny."""
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
                and not self.force_simt_gemm):
            if a.shape[0] <= self.skinny_max_tokens and w.shape[0] <= self.skinny_max_rows \
                    and not self.force_tcgen05_gemm:
                self.gemm_tn_skinny(a, w, out, swiglu8, early=early)   # a few tokens: bound by streaming the weights
            else:
                self.gemm_tn_tcgen05(a, w, out, swiglu8=swiglu8)
        else:
            if swiglu8:
                raise ShapeError("the fused SwiGLU epilogue exists in the bfloat16 tensor-core kernels only")
            self.gemm_tn_simt(a, w, out)

    def paged_attention_rows(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv, hd,
                             page_size, scale, window=0):
        """bfloat16 tensor-core attention for a ragged batch; work: int32 [n, 2] (entry, tile of 64 rows)."""
        self._check(self.lib.srlm_paged_attention_rows(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), C.c_int(block_table.stride(0)),
            _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]), C.c_int(nq), C.c_int(nkv), C.c_int(hd),
            C.c_int(page_size), C.c_float(scale), C.c_int(window or 0), _stream()), "paged_attention_rows")

    def paged_attention_rows_tma(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv, hd,
                                 page_size, scale, window=0):
        """Rows-split attention with TMA page loads; work: int32 [n, 2] (entry, tile of 128 rows)."""
        err = self._gemm_state(q.device)[1]
        self._check(self.lib.srlm_paged_attention_rows_tma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
            C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
            C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            _ptr(err), _stream()), "paged_attention_rows_tma")

    def paged_attention_prefill_tcgen05(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, work, nq, nkv,
                                        hd, page_size, scale, window=0, tiles_per_block=2, nsplit=1, kv_chunk=0,
                                        part_o=None, part_ml=None, sinks=None, mods=None):
        """Rows-split attention on tcgen05 tensor cores with accumulators in tensor memory (head size
        128; page_size 8..64 a power of two, or a multiple of 128); work: int32 [n, 2] (entry, block of
        tiles_per_block x 128 rows), tiles_per_block 1 or 2.  nsplit > 1: the keys in slices of kv_chunk
        (a multiple of 128), a block each, added by a second kernel; part_o float32
        [n * 2 * nkv * nsplit * 128, 128] and part_ml [.., 2] are their workspace."""
        err = self._gemm_state(q.device)[1]
        if mods is not None:        # (head_scale, pen_weight, pen_rate[, softcap]): float32 [nq] each or None, and a number; see paged_attention_general
            self._check(self.lib.srlm_paged_attention_prefill_tcgen05_mods(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
                C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
                C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
                C.c_int(tiles_per_block), C.c_int(nsplit), C.c_int(kv_chunk), _ptr(part_o), _ptr(part_ml), _ptr(sinks),
                _ptr(mods[0]), _ptr(mods[1]), _ptr(mods[2]), C.c_float(mods[3] if len(mods) > 3 and mods[3] else 0.0),
                _ptr(err), _stream()), "paged_attention_prefill_tcgen05")
        elif sinks is not None:     # float32 [nq]: one more term exp(sink) in each head's softmax denominator
            self._check(self.lib.srlm_paged_attention_prefill_tcgen05_sinks(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
                C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
                C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
                C.c_int(tiles_per_block), C.c_int(nsplit), C.c_int(kv_chunk), _ptr(part_o), _ptr(part_ml), _ptr(sinks),
                _ptr(err), _stream()), "paged_attention_prefill_tcgen05")
        else:
            self._check(self.lib.srlm_paged_attention_prefill_tcgen05(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
                C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), _ptr(work), C.c_int(work.shape[0]),
                C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
                C.c_int(tiles_per_block), C.c_int(nsplit), C.c_int(kv_chunk), _ptr(part_o), _ptr(part_ml), _ptr(err),
                _stream()), "paged_attention_prefill_tcgen05")
        if nsplit > 1:
            self.launches += 1           # the kernel that adds the slices

    @staticmethod
    def prefill_attention_plan(rows, kv_lens, nkv: int, sms: int):
        """(tiles_per_block, nsplit, kv_chunk) for the tensor-memory attention kernel on entries of
        ``rows`` rows (tokens x query heads per KV head) and ``kv_lens`` keys.  The choice goes by a
        model of the kernel's time, fitted to measurements on B200 (one portion of 481 to 512 tokens behind
        1,024 and 8,192 cached ones, 32 and 40 heads over 8 KV heads), in microseconds: a block of one row
        tile takes 7.8 + 1.75 a key tile, a block of two row tiles 11.7 + 1.92 a key tile (the tensor core
        works on one tile while the other is in its softmax), blocks run in rounds of one per SM, and
        cutting the keys into slices adds 11 (the slices' outputs go through a workspace and a second
        kernel).  So: two row tiles a block when the rows fill the SMs or one-tile blocks would need a
        round more; key slices for a portion behind a long context (512 tokens behind 8,192: 126.6 us in
        one-tile blocks, 88.6 us in two slices of two-tile blocks)."""
        two_tile_blocks = sum((r + 255) // 256 for r in rows) * nkv
        one_tile_blocks = sum((r + 127) // 128 for r in rows) * nkv
        key_tiles = max(1, (max(kv_lens) + 127) // 128)
        rounds = lambda blocks: -(-blocks // max(1, sms))
        best = (rounds(one_tile_blocks) * (key_tiles * 1.75 + 7.8), 1, 1)
        for s in range(1, min(16, max(1, key_tiles // 2)) + 1):
            per_slice = -(-key_tiles // s)
            t = rounds(two_tile_blocks * s) * (per_slice * 1.92 + 11.7) + (11.0 if s > 1 else 0.0)
            if t < best[0] - 1e-9:
                best = (t, 2, s)
        _, tiles, s = best
        if s == 1:
            return tiles, 1, 0
        chunk = -(-key_tiles // s) * 128
        return tiles, -(-key_tiles * 128 // chunk), chunk

    def paged_attention_keys(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, n_entries, nq, nkv, hd,
                             page_size, scale, window, kv_chunk, nsplit, part_o=None, part_ml=None):
        """bfloat16 tensor-core attention when every entry has at most 16 rows (decode); keys in nsplit slices."""
        counters = None
        if nsplit > 1:
            counters = getattr(self, "_slice_counters", None)
            if counters is None or counters.device != q.device:
                counters = self._slice_counters = torch.zeros(1 << 16, dtype=torch.int32, device=q.device)
            if n_entries * nkv > counters.numel():
                raise ShapeError(f"paged_attention_keys: {n_entries} entries x {nkv} KV heads exceed the counters")
        self._check(self.lib.srlm_paged_attention_keys(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), C.c_int(block_table.stride(0)),
            _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries), C.c_int(nq), C.c_int(nkv), C.c_int(hd),
            C.c_int(page_size), C.c_float(scale), C.c_int(window or 0), C.c_int(kv_chunk), C.c_int(nsplit),
            _ptr(part_o), _ptr(part_ml), _ptr(counters), _stream()), "paged_attention_keys")

    def _slice_counter_buffer(self, device, need):
        counters = getattr(self, "_slice_counters", None)
        if counters is None or counters.device != device:
            counters = self._slice_counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        if need > counters.numel():
            raise ShapeError(f"attention: {need} (entry, KV head) pairs exceed the slice counters")
        return counters

    def paged_attention_decode_tma(self, q, k_cache, v_cache, out, block_table, cu_q, kv_lens, n_entries, nq, nkv,
                                   hd, page_size, scale, window, kv_chunk, nsplit, part_o=None, part_ml=None,
                                   cluster=True):
        """Decode attention with TMA page loads (head_dim a multiple of 64; page_size 8, 16, 32 or a
        multiple of 64); same contract as paged_attention_keys.  cluster: up to 8 slices are merged
        through the distributed shared memory of a thread-block cluster (part_o / part_ml not needed)."""
        counters = self._slice_counter_buffer(q.device, n_entries * nkv) if nsplit > 1 else None
        err = self._gemm_state(q.device)[1]
        self._check(self.lib.srlm_paged_attention_decode_tma(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]), _ptr(block_table),
            C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries), C.c_int(nq),
            C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            C.c_int(kv_chunk), C.c_int(nsplit), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            C.c_int(1 if cluster else 0), _ptr(err), _stream()), "paged_attention_decode_tma")

    def paged_attention_decode_fused(self, qkv, q_norm_w, k_norm_w, eps, cos, sin, write_kv, k_cache, v_cache, out,
                                     block_table, cu_q, kv_lens, n_entries, nq, nkv, hd, page_size, scale, window,
                                     kv_chunk, nsplit, part_o=None, part_ml=None, cluster=True):
        """paged_attention_decode_tma with the step before it folded in: q and the step's new keys and
        values are read from qkv [tokens, (nq + 2 nkv) * hd], normalised per head (weights may be None)
        and rotated (cos / sin [tokens, hd/2], pairs (i, i + hd/2)) inside the kernel; with write_kv the
        new keys and values are written to the cache.  head_dim 64, 128 or 256."""
        counters = self._slice_counter_buffer(qkv.device, n_entries * nkv) if nsplit > 1 else None
        err = self._gemm_state(qkv.device)[1]
        self._check(self.lib.srlm_paged_attention_decode_fused(
            _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), C.c_float(eps), _ptr(cos), _ptr(sin),
            C.c_int(int(write_kv)), _ptr(k_cache), _ptr(v_cache), _ptr(out), C.c_longlong(k_cache.shape[0]),
            _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(cu_q), _ptr(kv_lens), C.c_int(n_entries),
            C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(page_size), C.c_float(scale), C.c_int(window or 0),
            C.c_int(kv_chunk), C.c_int(nsplit), _ptr(part_o), _ptr(part_ml), _ptr(counters),
            C.c_int(1 if cluster else 0), _ptr(err), _stream()), "paged_attention_decode_fused")

    @staticmethod
    def attention_split(n_entries: int, nkv: int, max_kv: int, max_slices: int = 32):
        """(nsplit, kv_chunk) for the keys-split kernels: as many blocks as run at the same time (two per
        SM) and no more -- a few blocks left over for a second wave would double the time -- in slices of
        whole tiles."""
        tiles = max(1, (max_kv + 63) // 64)
        nsplit = max(1, min(tiles, 2 * KernelLibrary.SMS // max(1, n_entries * nkv), max_slices))
        chunk = -(-tiles // nsplit) * 64
        nsplit = -(-tiles * 64 // chunk)
        return nsplit, chunk

    def _decode_plan(self, ctx, nkv, hd, n_entries=None, kv_bound=None):
        """(nsplit, kv_chunk, cluster, part_o, part_ml) for the TMA decode kernel on the batch of ctx, or on
        ``n_entries`` of its entries whose keys number at most ``kv_bound``."""
        n_entries = ctx.n_entries if n_entries is None else n_entries
        kv_bound = ctx.kv_bound if kv_bound is None else kv_bound
        nsplit, chunk = self.attention_split(n_entries, nkv, kv_bound)
        # Up to 8 slices merge inside a thread-block cluster, which saves the round trip through global
        # memory (6 to 8 us measured); more slices pay only when each of the 8 would have many more
        # tiles to walk (about 1 us a tile).
        cluster = False
        if self.cluster_decode_merge and nsplit > 1:
            n8, chunk8 = self.attention_split(n_entries, nkv, kv_bound, max_slices=8)
            if chunk8 - chunk <= 7 * 64:
                nsplit, chunk, cluster = n8, chunk8, True
        part_o = part_ml = None
        if nsplit > 1 and not cluster:
            part_o = ctx.workspace.get("attn.part_o", n_entries * nkv * nsplit * 16, hd, torch.float32, reserve=0)
            part_ml = ctx.workspace.get("attn.part_ml", n_entries * nkv * nsplit * 16, 2, torch.float32,
                                        reserve=0)
        return nsplit, chunk, cluster, part_o, part_ml

    def attention_from_projection(self, ctx, qkv, k_cache, v_cache, out, block_table, q_norm_w, k_norm_w, eps,
                                  rotation, write_kv, nq, nkv, hd, page_size, scale, window=0) -> bool:
        """Decode steps: per-head norm, rotation, append to the cache and attention over the cache in one
        kernel, straight from the q/k/v projection's output.  rotation: a parts.base.Rotation or None.
        Returns False (and does nothing) when the batch, the sizes or the rotation (half-split pairs over
        the whole head) are not the ones that kernel takes; the caller then runs the steps one by one."""
        g = nq // nkv
        if (not self.fuse_decode_attention or qkv.dtype != torch.bfloat16 or ctx.max_q_len * g > 16
                or hd not in (64, 128, 256) or rotation is None or rotation.interleaved
                or 2 * rotation.pairs != hd
                or self.force_simt_attention or self.force_cp_async_decode
                or not self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size))):
            return False
        nsplit, chunk, cluster, part_o, part_ml = self._decode_plan(ctx, nkv, hd)
        self.paged_attention_decode_fused(qkv, q_norm_w, k_norm_w, eps, rotation.cos, rotation.sin, write_kv,
                                          k_cache, v_cache, out,
                                          block_table, ctx.cu_q, ctx.kv_lens, ctx.n_entries, nq, nkv, hd,
                                          page_size, scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
        return True

    def sinks_on_tcgen05(self, ctx, dtype, nq, nkv, hd, dv, page_size) -> bool:
        """Whether paged_attention(..., sinks=...) can serve this step: only its tensor-memory rows kernel knows
        sinks (head size 128 for keys and values, bfloat16, some entry of more than 16 rows)."""
        return (dtype == torch.bfloat16 and hd == dv and ctx.max_q_len * (nq // nkv) > 16
                and not self.force_simt_attention and not self.force_mma_sync_prefill and self.sinks_in_tcgen05_prefill
                and bool(self.lib.srlm_attention_prefill_tcgen05_takes(C.c_int(hd), C.c_int(page_size))))

    def paged_attention(self, ctx, q, k_cache, v_cache, out, block_table, nq, nkv, hd, page_size, scale,
                        window=0, sinks=None, mods=None):
        """The product path's attention over the cache for the batch of ``ctx``: tensor cores for
        bfloat16 (keys-split when every entry is a few rows, rows-split otherwise), float32 FMA for
        the float32 path.  sinks (float32 [nq]), and mods (head_scale, pen_weight, pen_rate: the per-head score
        changes of paged_attention_general): only where sinks_on_tcgen05 says so; every entry then goes
        to the rows kernel."""
        if (sinks is not None or mods is not None) and not self.sinks_on_tcgen05(ctx, q.dtype, nq, nkv, hd, hd, page_size):
            raise ShapeError("paged_attention: sinks and score changes are served by the tensor-memory rows kernel only")
        special = sinks is not None or mods is not None
        if q.dtype != torch.bfloat16 or hd % 16 or hd > 256 or self.force_simt_attention:
            self.paged_attention_simt(q, k_cache, v_cache, out, block_table, ctx.entry_of_token, ctx.positions,
                                      nq, nkv, hd, page_size, scale, window)
            return
        g = nq // nkv

        def keys_split(lo, hi):
            """Entries lo..hi-1, each of at most 16 rows (tokens x heads per KV head): the kernels that split
            the keys over blocks.  They index the step's q and out by the token offsets in cu_q, so a run of
            entries is served by handing them the run's part of cu_q, kv_lens and the block table."""
            n = hi - lo
            whole = lo == 0 and hi == ctx.n_entries
            bound = ctx.kv_bound if whole else max(ctx.host["kv_lens"][lo:hi])
            cu, kvl, table = ctx.cu_q[lo:hi + 1], ctx.kv_lens[lo:hi], block_table[lo:hi]
            if self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size)) and not self.force_cp_async_decode:
                nsplit, chunk, cluster, part_o, part_ml = self._decode_plan(ctx, nkv, hd, n, bound)
                self.paged_attention_decode_tma(q, k_cache, v_cache, out, table, cu, kvl, n, nq, nkv, hd, page_size,
                                                scale, window, chunk, nsplit, part_o, part_ml, cluster=cluster)
                return
            nsplit, chunk = self.attention_split(n, nkv, bound)
            part_o = part_ml = None
            if nsplit > 1:
                part_o = ctx.workspace.get("attn.part_o", n * nkv * nsplit * 16, hd, torch.float32, reserve=0)
                part_ml = ctx.workspace.get("attn.part_ml", n * nkv * nsplit * 16, 2, torch.float32, reserve=0)
            self.paged_attention_keys(q, k_cache, v_cache, out, table, cu, kvl, n, nq, nkv, hd, page_size, scale,
                                      window, chunk, nsplit, part_o, part_ml)

        if ctx.max_q_len * g <= 16:
            keys_split(0, ctx.n_entries)
            return
        # A mixed step: decoding requests (a row or a few) beside portions of prompts.  A row tile of the
        # rows-split kernels would be all but empty for a decoding request and would walk its keys alone,
        # one block per KV head; so the decoding requests at the head and at the tail of the batch (the
        # scheduler puts them first) go to the keys-split kernel, the rest to the rows-split one.
        q_lens = ctx.host["q_lens"]
        n = ctx.n_entries
        head = 0
        while head < n and q_lens[head] * g <= 16:
            head += 1
        tail = n
        while tail > head and q_lens[tail - 1] * g <= 16:
            tail -= 1
        # Worth a launch of its own only when the decoding requests would fill a round of blocks of the
        # rows-split kernel by themselves (one block per request and KV head) and their contexts are of
        # similar length: the two launches run one after the other, and the keys-split one lasts as long
        # as its longest request, while row tiles of all kinds share the SMs in one launch.  Measured at
        # 8B / 14B sizes: 31 decoding requests of 1,500 tokens beside a 481-token portion, 7 % / 2 % of
        # the step faster in two launches; 32 requests of 128 to 3,200 tokens, 1.5 % slower.
        short = list(range(head)) + list(range(tail, n))
        enough = self.sm_count(q.device) if self.split_mixed_min_blocks is None else self.split_mixed_min_blocks
        if not special and self.split_mixed_attention and ctx.max_q_len > 1 and short and len(short) * nkv >= enough:
            lens = [ctx.host["kv_lens"][e] for e in short]
            if max(lens) * len(lens) > 1.5 * sum(lens):
                short = []
        else:
            short = []
        if not short:
            head, tail = 0, n
        if head > 0:
            keys_split(0, head)
        if tail < n:
            keys_split(tail, n)
        rows_entries = range(head, tail)
        def work_list(rows_per_block):
            if ctx.max_q_len == 1:
                # decode steps (more than 16 query heads per KV head): the list depends on the number of
                # entries alone, so it is made once and kept on the device; such steps are recorded into
                # CUDA graphs, and a recording must not hold a copy from a buffer that lives for one step
                lists = self.__dict__.setdefault("_decode_work_lists", {})
                key = (q.device, ctx.n_entries, g, rows_per_block)      # (every entry: head = 0, tail = n)
                if key not in lists:
                    tiles = (g + rows_per_block - 1) // rows_per_block
                    lists[key] = torch.tensor([(e, t) for e in range(ctx.n_entries) for t in range(tiles)],
                                              dtype=torch.int32).to(q.device)
                return lists[key]
            work = ctx.tables.get(("attention_rows_work", g, rows_per_block))
            if work is None:
                # the last row blocks of an entry see the most keys: they go first, so that the long
                # blocks do not start when the short ones have already left the GPU half empty
                pairs = [(e, t) for e in rows_entries
                         for t in reversed(range((q_lens[e] * g + rows_per_block - 1) // rows_per_block))]
                pairs.sort(key=lambda et: -(ctx.host["starts"][et[0]] + (et[1] + 1) * rows_per_block // g))
                work = torch.tensor(pairs, dtype=torch.int32).pin_memory().to(q.device, non_blocking=True)
                ctx.tables[("attention_rows_work", g, rows_per_block)] = work
            return work

        if (self.lib.srlm_attention_prefill_tcgen05_takes(C.c_int(hd), C.c_int(page_size))
                and not self.force_mma_sync_prefill):
            rows = [q_lens[e] * g for e in rows_entries]
            # a decode step may be replayed from a CUDA graph with longer contexts than it was recorded
            # with: its plan goes by the bound that is part of the graph's identity
            lens = [ctx.kv_bound] if ctx.max_q_len == 1 else [ctx.host["kv_lens"][e] for e in rows_entries]
            tiles, nsplit, chunk = self.prefill_attention_plan(rows, lens, nkv, self.sm_count(q.device))
            if not self.split_prefill_keys:
                nsplit, chunk = 1, 0
            work = work_list(128 * tiles)
            part_o = part_ml = None
            if nsplit > 1:
                slabs = work.shape[0] * 2 * nkv * nsplit * 128
                part_o = ctx.workspace.get("attn.rows_part_o", slabs, hd, torch.float32, reserve=0)
                part_ml = ctx.workspace.get("attn.rows_part_ml", slabs, 2, torch.float32, reserve=0)
            self.paged_attention_prefill_tcgen05(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens, work,
                                                 nq, nkv, hd, page_size, scale, window, tiles, nsplit, chunk, part_o,
                                                 part_ml, sinks=sinks, mods=mods)
            return
        tma = (hd in (64, 128) and self.lib.srlm_attention_decode_tma_takes(C.c_int(hd), C.c_int(page_size))
               and not self.force_cp_async_decode)
        if tma:
            self.paged_attention_rows_tma(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens,
                                          work_list(128), nq, nkv, hd, page_size, scale, window)
        else:
            self.paged_attention_rows(q, k_cache, v_cache, out, block_table, ctx.cu_q, ctx.kv_lens, work_list(64),
                                      nq, nkv, hd, page_size, scale, window)

    # ---- blocks that norm on both sides of a sublayer --------------------------------
    def gated_postnorm_add(self, residual, sub, gate, gate_bias, post_w, eps, next_w=None, next_eps=0.0,
                           next_out=None):
        """residual += post_w * rms_norm(sub * sigmoid(gate + gate_bias)); with next_out also
        next_out = next_w * rms_norm(residual).  residual float32 [T, H]; sub, gate (may be None) and
        next_out in the activation dtype; the weights float32 [H]."""
        T, H = residual.shape
        if residual.dtype != torch.float32 or tuple(sub.shape) != (T, H) or (gate is not None and gate.dtype != sub.dtype):
            raise ShapeError(f"gated_postnorm_add: residual {tuple(residual.shape)} {residual.dtype}, sub {tuple(sub.shape)}")
        self._check(self.lib.srlm_gated_postnorm_add(
            _ptr(residual), _ptr(sub), _ptr(gate), _ptr(gate_bias), _ptr(post_w), C.c_float(eps), _ptr(next_w),
            C.c_float(next_eps), _ptr(next_out), dtype_code(sub.dtype), C.c_int(T), C.c_int(H), _stream()),
            "gated_postnorm_add")

    # ---- attention with separate key and value sizes ---------------------------------------
    GENERAL_ROWS = 16        # rows (tokens x query heads of a KV head) of a block of the general attention kernel

    def paged_attention_general(self, ctx, q, k_cache, v_cache, out, block_table, sinks, nq, nkv, dk, dv, scale,
                                window=0, head_scale=None, penalty=None, gate=None, softcap=None):
        """Causal attention of the batch of ``ctx`` over pages whose keys have dk and whose values have dv
        elements (v_cache None: the values are the keys' first dv elements).  q float32 [T, nq * dk];
        k_cache [pages, nkv, page_size, dk]; out [T, nq * dv], float32 or the cache's dtype; sinks float32
        [nq] or None: one more term exp(sink) in each head's softmax denominator.  head_scale float32 [nq] or
        None: a factor per head on the scaled scores.  penalty (weight, rate), float32 [nq] each, or None:
        weight * ln(1 + rate * distance to the key) is taken off the score.  softcap (a number) or None: the scaled
        score s becomes softcap * tanh(s / softcap), ahead of the penalty.  window > 0: a query sees itself
        and the window - 1 keys before it.  gate (float32 tensor [T, >= column + nq], column) or None: head h of
        token t is multiplied by the logistic of tensor[t, column + h] as it is written.

        A bfloat16 cache: the tensor-core forms (attention_general_mma.cu) when they take the sizes -- the
        decode form for steps of at most four tokens an entry (keys in slices, as many blocks as run at the
        same time, added by a second kernel), the rows form for prompts, portions and mixed steps.  Else
        float32 arithmetic: a bfloat16 decode step in key slices too; the float32 path always one block per
        16 rows, whose sums do not depend on the batch."""
        if q.dtype != torch.float32:
            raise ShapeError("paged_attention_general: float32 queries")
        n = ctx.n_entries
        g = nq // nkv
        mods = (_ptr(head_scale), _ptr(penalty[0] if penalty else None), _ptr(penalty[1] if penalty else None),
                C.c_float(softcap or 0.0))
        if gate is not None:
            logits, column = gate
            if logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1 or logits.shape[1] < column + nq:
                raise ShapeError("paged_attention_general: the gate's logits are float32 columns of a row-major tensor")
            gate_args = (C.c_void_p(logits.data_ptr() + 4 * column), C.c_longlong(logits.stride(0)))
        else:
            gate_args = (C.c_void_p(0), C.c_longlong(0))
        bf16 = k_cache.dtype == torch.bfloat16
        tensor_cores = bf16 and self.general_attention_on_tensor_cores
        from_keys = C.c_int(int(v_cache is None))
        # a decode step: one to four tokens an entry.  Its keys are cut into slices, as many blocks as run at once.
        if (tensor_cores and ctx.max_q_len <= 4
                and self.lib.srlm_attention_general_decode_takes(C.c_int(dk), C.c_int(dv), from_keys)):
            rows_padded = (ctx.max_q_len * g + 15) // 16 * 16
            # with a window the slices lie over the keys a row tile can see, not over the whole context
            span = min(ctx.kv_bound, window + ctx.max_q_len + 64) if window else ctx.kv_bound
            nsplit, chunk = self.attention_split(n, nkv * (rows_padded // 16), span, max_slices=64)
            if not self.split_general_attention:
                nsplit, chunk = 1, 0
            part_o = part_ml = None
            if nsplit > 1:
                part_o = ctx.workspace.get("attn.general_part_o", n * nkv * nsplit * rows_padded, dv, torch.float32,
                                           reserve=0)
                part_ml = ctx.workspace.get("attn.general_part_ml", n * nkv * nsplit * rows_padded, 2, torch.float32,
                                            reserve=0)
            self._check(self.lib.srlm_paged_attention_general_decode(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), dtype_code(out.dtype), _ptr(block_table),
                C.c_int(block_table.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.kv_lens), _ptr(sinks), C.c_int(n),
                C.c_int(ctx.max_q_len), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv), C.c_int(k_cache.shape[2]),
                C.c_float(scale), C.c_int(window or 0), C.c_int(nsplit), C.c_int(chunk), _ptr(part_o), _ptr(part_ml),
                *mods, *gate_args, _stream()), "paged_attention_general_decode")
            if nsplit > 1:
                self._check(self.lib.srlm_attention_general_merge(
                    _ptr(part_o), _ptr(part_ml), _ptr(out), dtype_code(out.dtype), _ptr(ctx.cu_q), C.c_int(n),
                    C.c_int(nq), C.c_int(nkv), C.c_int(dv), C.c_int(nsplit), C.c_int(rows_padded), *gate_args, _stream()),
                    "attention_general_merge")
            return
        decode = ctx.max_q_len * g <= self.GENERAL_ROWS
        if (tensor_cores and not decode
                and self.lib.srlm_attention_general_mma_takes(C.c_int(dk), C.c_int(dv), from_keys)):
            # prompts and their portions: bfloat16 tensor cores (the queries are rounded as they are loaded)
            self._check(self.lib.srlm_paged_attention_general_mma(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), dtype_code(out.dtype), _ptr(block_table),
                C.c_int(block_table.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.kv_lens), _ptr(sinks), C.c_int(n),
                C.c_int(ctx.max_q_len), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv),
                C.c_int(k_cache.shape[2]), C.c_float(scale), C.c_int(window or 0), *mods, *gate_args, _stream()),
                "paged_attention_general_mma")
            return
        # float32, and sizes the tensor-core forms do not take: float32 arithmetic; a bfloat16 decode step in slices
        nsplit, chunk, part_o, part_ml = 1, 0, None, None
        if bf16 and decode and self.split_general_attention:
            span = min(ctx.kv_bound, window + ctx.max_q_len + 64) if window else ctx.kv_bound
            nsplit, chunk = self.attention_split(n, nkv, span, max_slices=64)
            if nsplit > 1:
                part_o = ctx.workspace.get("attn.general_part_o", n * nkv * nsplit * self.GENERAL_ROWS, dv,
                                           torch.float32, reserve=0)
                part_ml = ctx.workspace.get("attn.general_part_ml", n * nkv * nsplit * self.GENERAL_ROWS, 2,
                                            torch.float32, reserve=0)
        self._check(self.lib.srlm_paged_attention_general(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), dtype_code(k_cache.dtype), dtype_code(out.dtype),
            _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.kv_lens), _ptr(sinks),
            C.c_int(n), C.c_int(ctx.max_q_len), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv),
            C.c_int(k_cache.shape[2]), C.c_float(scale), C.c_int(window or 0), C.c_int(nsplit), C.c_int(chunk),
            _ptr(part_o), _ptr(part_ml), *mods, *gate_args, _stream()), "paged_attention_general")
        if nsplit > 1:
            self.launches += 1           # the kernel that adds the slices

    def attention_bias_append(self, proj, bias, q_out, k_cache, v_cache, kv_slot, nq, nkv, dk, dv, v_keep=None,
                              lam=None, mix_mode=0, write_kv=True, rotation=None):
        """From a stacked q | k | v projection [T, >= nq dk + nkv (dk + dv)]: q + bias to q_out (float32, or
        bfloat16 for the kernels that take their queries so), k + bias
        and v + bias to the pages.  mix_mode 1 also keeps v in v_keep (float32 [T, nkv dv]); mix_mode 2 writes
        (1 - lam) v + lam v_keep instead of v (lam: float32 [1] on the device).  rotation (parts.base.Rotation) or
        None: the first 2 * pairs elements of every q and k head are turned, behind the bias, by the step's angles.
        write_kv False without value mixing: proj holds the q columns alone."""
        T = proj.shape[0]
        pairs = rotation.pairs if rotation is not None else 0
        self._check(self.lib.srlm_attention_bias_append(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), _ptr(bias), _ptr(q_out),
            dtype_code(q_out.dtype), _ptr(k_cache), _ptr(v_cache), dtype_code(k_cache.dtype), _ptr(kv_slot), _ptr(v_keep), _ptr(lam), C.c_int(mix_mode),
            C.c_int(int(write_kv)), C.c_int(T), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv),
            C.c_int(k_cache.shape[2]), _ptr(rotation.cos if pairs else None), _ptr(rotation.sin if pairs else None),
            C.c_int(pairs), C.c_int(int(bool(pairs and rotation.interleaved))), _stream()), "attention_bias_append")

    def attention_unit_norm_append(self, proj, eps, q_out, k_cache, v_cache, kv_slot, nq, nkv, dk, dv, write_kv=True):
        """From a stacked q | k | v (| more) projection [T, >= nq dk + nkv (dk + dv)]: every q and k head divided by
        sqrt(mean(x^2) + eps) in float32 (eps None: as projected); q to q_out (float32 or bfloat16), k and v to the pages."""
        self._check(self.lib.srlm_attention_unit_norm_append(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), C.c_float(eps if eps else 0.0), _ptr(q_out),
            dtype_code(q_out.dtype), _ptr(k_cache), _ptr(v_cache), dtype_code(k_cache.dtype), _ptr(kv_slot),
            C.c_int(int(write_kv)), C.c_int(proj.shape[0]), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv),
            C.c_int(k_cache.shape[2]), _stream()), "attention_unit_norm_append")

    def softcap(self, x, cap):
        """x <- cap * tanh(x / cap), float32 in place."""
        if x.dtype != torch.float32:
            raise ShapeError("softcap: float32 values")
        self._check(self.lib.srlm_softcap(_ptr(x), C.c_float(cap), C.c_longlong(x.numel()), _stream()), "softcap")

    # ---- routed experts ----------------------------------------------------------------------
    def moe_tile_rows(self) -> int:
        return int(self.lib.srlm_moe_tile_rows())

    @staticmethod
    def _columns(t, column, width):
        """(pointer, leading dimension) of the float32 columns [column, column + width) of a row-major tensor."""
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1 or t.shape[1] < column + width:
            raise ShapeError("float32 columns of a row-major CUDA tensor are wanted")
        return C.c_void_p(t.data_ptr() + 4 * column), C.c_longlong(t.stride(0))

    ROUTER_SCORING = {"softmax_of_chosen": 0, "logistic": 1, "softmax_over_all": 2}

    def moe_route(self, logits, bias, top, choice, weight, column=0, experts=None, scoring="softmax_of_chosen",
                  groups=(1, 1)):
        """logits float32 [T, E] (+ bias float32 [E]) -> choice int32 [T, top], the experts with the largest
        logits (ties: the lowest index), and weight float32 [T, top]: the softmax over the chosen logits, or
        (scoring "logistic") the logistic of each chosen logit, not renormalised, or (scoring "softmax_over_all") the
        softmax over all logits, renormalised over the chosen ones; then groups = (count, kept): the experts form
        ``count`` equal groups of neighbours and only experts of the ``kept`` groups with the largest scores are chosen.
        column / experts: the logits are those columns of a wider tensor."""
        T = logits.shape[0]
        E = logits.shape[1] - column if experts is None else experts
        if choice.dtype != torch.int32 or weight.dtype != torch.float32:
            raise ShapeError("moe_route: float32 logits and weights, int32 choices")
        ptr, ld = self._columns(logits, column, E)
        self._check(self.lib.srlm_moe_route(ptr, ld, _ptr(bias), C.c_int(T), C.c_int(E),
                                            C.c_int(top), _ptr(choice), _ptr(weight),
                                            C.c_int(self.ROUTER_SCORING[scoring]), C.c_int(groups[0]), C.c_int(groups[1]),
                                            _stream()), "moe_route")

    def moe_sort_routes(self, tokens, experts) -> bool:
        """Whether moe_sort(..., route=...) routes a step of this many tokens itself."""
        return bool(self.lib.srlm_moe_sort_routes(C.c_int(tokens), C.c_int(experts)))

    def moe_sort(self, choice, experts, offsets, tiles, pair_of_row, row_of_pair, tile_rows=0, group_of_tile=None,
                 route=None, scoring="softmax_of_chosen", groups=(1, 1)):
        """The (token, choice) pairs ordered by expert: offsets / tiles int32 [experts + 1] (first row and first
        tile of each expert), pair_of_row / row_of_pair int32 [pairs].  tile_rows > 0: every expert's rows start at
        a multiple of tile_rows; pair_of_row then covers all rows of group_of_tile's tiles (-1: a row without a
        pair) and group_of_tile int32 [tiles] names each tile's expert (-1: none).  route (logits, column, bias,
        weight): the kernel first routes the tokens itself, as moe_route does, and writes choice and weight."""
        if route is not None:
            logits, column, bias, weight = route
            ptr, ld = self._columns(logits, column, experts)
            routing = (ptr, ld, _ptr(bias), C.c_int(choice.shape[1]), _ptr(weight))
        else:
            routing = (C.c_void_p(0), C.c_longlong(0), C.c_void_p(0), C.c_int(0), C.c_void_p(0))
        self._check(self.lib.srlm_moe_sort(
            _ptr(choice), C.c_int(choice.numel()), C.c_int(experts), _ptr(offsets), _ptr(tiles), _ptr(pair_of_row),
            _ptr(row_of_pair), C.c_int(tile_rows), _ptr(group_of_tile),
            C.c_int(group_of_tile.numel() if group_of_tile is not None else 0),
            C.c_int(pair_of_row.numel()), *routing, C.c_int(self.ROUTER_SCORING[scoring]), C.c_int(groups[0]),
            C.c_int(groups[1]), _stream()), "moe_sort")

    GROUPED_TILE = 128       # token rows of a tile of the grouped tensor-memory product (one SM a tile)
    GROUPED_PAIR_TILE = 256  # ... of its pair form (two SMs on 256 weight rows x 256 tokens)

    def grouped_tile_rows(self, pairs: int, experts: int, weight_elements: int) -> int:
        """The token tile of the grouped tensor-memory product for a step of ``pairs`` rows over ``experts`` groups
        whose first weight matrix has ``weight_elements`` elements a group: 256 (pairs of SMs) once an expert has 512
        rows on average (so that about an eighth of the tiles' rows is padding) and 16 Mi weight elements; else 128.
        Measured at 8,192 rows over 16 experts: 2,048 x 2,048 a group 0.76 ms in pairs against 0.68 ms for the eight
        products of four layers, 4,096 x 4,096 a group 1.32 against 1.85 ms."""
        big = pairs >= 512 * experts and weight_elements >= 16 << 20
        return self.GROUPED_PAIR_TILE if self.grouped_pairs and big else self.GROUPED_TILE

    def moe_gather_rows(self, x, pair_of_row, pairs_per_token, out, pair_scale=None):
        """out[row] = x[pair_of_row[row] // pairs_per_token] (bfloat16 rows; zeros where pair_of_row is -1), times
        pair_scale[pair] (float32, one number a pair) when given."""
        self._check(self.lib.srlm_moe_gather_rows(_ptr(x), C.c_longlong(x.stride(0)), _ptr(pair_of_row),
                                                  C.c_int(pairs_per_token), _ptr(out), C.c_int(out.shape[0]),
                                                  C.c_int(out.shape[1]), _ptr(pair_scale), _stream()), "moe_gather_rows")

    def gemm_tn_tcgen05_grouped(self, x, w, out, group_of_tile, glu=False, limit=0.0, alpha=0.0, tile_rows=128, act=None):
        """out[r] = x[r] . w[group of r's tile]^T on the persistent tensor-memory kernel: x [rows, K] bfloat16 in tiles
        of tile_rows rows (128, or 256: pairs of SMs), w [groups, N, K]; a tile whose group is negative is skipped.
        glu: w's rows in blocks of 8 gate and 8 up rows, out [rows, N / 2] = the clamped GLU.  act "gelu" (without glu):
        out = the exact gelu of the product."""
        rows, K = x.shape
        G, N, _ = w.shape
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[2] != K or group_of_tile.numel() * tile_rows < rows:
            raise ShapeError(f"gemm_tcgen05_grouped: x {tuple(x.shape)}, w {tuple(w.shape)}, {group_of_tile.numel()} tiles")
        err = self._gemm_state(x.device)[1]
        self._check(self.lib.srlm_gemm_tn_tcgen05_grouped(
            _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), C.c_int(rows), C.c_int(N), C.c_int(K),
            C.c_longlong(x.stride(0)), C.c_longlong(out.stride(0)), C.c_int(G), _ptr(group_of_tile), C.c_int(tile_rows),
            C.c_int(int(glu)),
            C.c_float(limit), C.c_float(alpha), C.c_int(self.PLAIN_ACTIVATIONS[act]), _ptr(err), _stream()),
            "gemm_tn_tcgen05_grouped")

    PLAIN_ACTIVATIONS = {None: 0, "gelu": 1}

    def moe_grouped(self, a, pair_of_row, pairs_per_token, w, out, offsets, tiles, glu=False, interleaved=False,
                    limit=0.0, alpha=0.0, pair_scale=None, act=None):
        """out[row] = a[row's token] . w[row's expert]^T for every row of the sorted pairs (pair_of_row None: row r
        of ``a`` is row r of ``out``).  w [experts, N, K]; glu: w [experts, 2 N, K] and out gets the clamped GLU of
        the gate and up halves (interleaved: in blocks of 8 gate rows and 8 up rows, else all gate rows first);
        limit 0: the plain GLU, gate * logistic(gate) * up.  pair_scale (float32, one number a pair; with glu): the
        gate and up sums of a row are multiplied by its pair's number ahead of the activation, which for experts
        without biases is the activation of the scaled input.  act "gelu" (without glu): out gets the exact gelu of
        the product."""
        E, rows, K = w.shape
        n, N = out.shape
        if a.shape[1] != K or rows != (2 * N if glu else N):
            raise ShapeError(f"moe_grouped: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (interleaved or not glu) and a.stride(0) % 8 == 0
                and self.grouped_products_on_tensor_cores
                and self.lib.srlm_moe_grouped_mma_takes(C.c_int(N), C.c_int(K), C.c_int(int(glu)))):
            self._check(self.lib.srlm_moe_grouped_mma(
                _ptr(a), C.c_longlong(a.stride(0)), _ptr(pair_of_row), C.c_int(pairs_per_token), _ptr(w), _ptr(out),
                dtype_code(out.dtype), C.c_longlong(out.stride(0)), _ptr(offsets), _ptr(tiles), C.c_int(n), C.c_int(E),
                C.c_int(N), C.c_int(K), C.c_int(int(glu)), C.c_float(limit), C.c_float(alpha), _ptr(pair_scale),
                C.c_int(self.PLAIN_ACTIVATIONS[act]), _stream()), "moe_grouped_mma")
            return
        self._check(self.lib.srlm_moe_grouped_simt(
            _ptr(a), dtype_code(a.dtype), C.c_longlong(a.stride(0)), _ptr(pair_of_row), C.c_int(pairs_per_token), _ptr(w),
            dtype_code(w.dtype), _ptr(out), dtype_code(out.dtype), C.c_longlong(out.stride(0)), _ptr(offsets), _ptr(tiles),
            C.c_int(n), C.c_int(E), C.c_int(N), C.c_int(K), C.c_int(int(glu)), C.c_int(int(interleaved)), C.c_float(limit),
            C.c_float(alpha), _ptr(pair_scale), C.c_int(self.PLAIN_ACTIVATIONS[act]), _stream()), "moe_grouped_simt")

    def moe_combine(self, rows, row_of_pair, weight, shared, out):
        """out[t] = sum over t's choices, in their order, of weight * rows[row of the pair] (+ shared[t]); weight
        None: the rows as they are; row_of_pair int32 [T, top]."""
        T, H = out.shape
        self._check(self.lib.srlm_moe_combine(
            _ptr(rows), dtype_code(rows.dtype), C.c_longlong(rows.stride(0)), _ptr(row_of_pair), _ptr(weight), _ptr(shared),
            _ptr(out), dtype_code(out.dtype), C.c_int(T), C.c_int(row_of_pair.numel() // T), C.c_int(H), _stream()), "moe_combine")

    def clamped_glu(self, gate_up, out, limit, alpha):
        """out [T, F] = g * logistic(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); gate_up
        [T, >= 2 F]: gate columns, then up columns (whatever follows them is not read)."""
        T, F = out.shape
        self._check(self.lib.srlm_clamped_glu(_ptr(gate_up), dtype_code(gate_up.dtype), C.c_longlong(gate_up.stride(0)),
                                              _ptr(out), dtype_code(out.dtype),
                                              C.c_int(T), C.c_int(F), C.c_float(limit), C.c_float(alpha), _stream()),
                    "clamped_glu")

    # ---- the selective scan ---------------------------------------------------------------------
    def scan_conv(self, ctx, xz, conv_w, conv_b, state, x_out, x_low, channels, N, taps):
        """x_out float32 [T, channels] = silu(causal convolution over time of xz's first ``channels`` columns + conv_b);
        the inputs ahead of an entry's first token are the slot's carried ones (state [slots, channels * (N + taps - 1)]:
        S, then the last taps - 1 inputs of every channel).  x_low: a second copy in bfloat16, or None."""
        self._check(self.lib.srlm_scan_conv(
            _ptr(xz), C.c_longlong(xz.stride(0)), _ptr(conv_w), _ptr(conv_b), _ptr(state), C.c_longlong(state.stride(0)),
            _ptr(ctx.entry_of_token), _ptr(ctx.cu_q), _ptr(ctx.slots), _ptr(x_out), _ptr(x_low),
            dtype_code(x_low.dtype) if x_low is not None else DT_F32, C.c_int(xz.shape[0]), C.c_int(channels), C.c_int(N),
            C.c_int(taps), _stream()), "scan_conv")

    def selective_scan(self, ctx, x, xz, dbc, b_off, dt_raw, dt_bias, A, D, state, out, channels, N, taps):
        """Token by token in every entry: dt = softplus(dt_raw + dt_bias); S <- exp(dt A) S + dt x B; out = (S C + D x)
        silu(z).  x, dt_raw float32 [T, channels]; xz float32 [T, >= 2 channels] (inputs of the convolution, then z);
        dbc float32 rows with B in columns [b_off, b_off + N) and C behind them; A float32 [channels, N]; the slots'
        S and carried inputs in ``state`` are renewed."""
        self._check(self.lib.srlm_selective_scan(
            _ptr(x), _ptr(xz), C.c_longlong(xz.stride(0)), _ptr(dbc), C.c_longlong(dbc.stride(0)), C.c_int(b_off),
            _ptr(dt_raw), _ptr(dt_bias), _ptr(A), _ptr(D), _ptr(state), C.c_longlong(state.stride(0)), _ptr(ctx.cu_q),
            _ptr(ctx.slots), _ptr(out), dtype_code(out.dtype), C.c_int(ctx.n_entries), C.c_int(ctx.max_q_len), C.c_int(channels), C.c_int(N),
            C.c_int(taps), _stream()), "selective_scan")

    def paired_rmsnorm_mean(self, a, wa, b, wb, eps, out):
        """out = (wa * rms_norm(a) + wb * rms_norm(b)) / 2, rows of [T, H]; a and b of one dtype."""
        T, H = out.shape
        if a.dtype != b.dtype or tuple(a.shape) != (T, H) or tuple(b.shape) != (T, H):
            raise ShapeError(f"paired_rmsnorm_mean: a {tuple(a.shape)} {a.dtype}, b {tuple(b.shape)} {b.dtype}")
        self._check(self.lib.srlm_paired_rmsnorm_mean(_ptr(a), _ptr(wa), _ptr(b), _ptr(wb), C.c_float(eps), _ptr(out),
                                                      dtype_code(a.dtype), dtype_code(out.dtype), C.c_int(T), C.c_int(H),
                                                      _stream()), "paired_rmsnorm_mean")

    # ---- blocks that norm after the sum, and their elementwise companions ---------------------------
    def postnorm_scale_add(self, residual, delta, weight, alpha, eps, unit_offset=False, out=None, terms=None):
        """residual <- w' * y / sqrt(mean(y^2) + eps) with y = alpha * residual + delta and w' = weight (or 1 + weight),
        in place (float32 [T, H]); delta [T, H] in float32 or the activation dtype, or None; ``out``: a copy of the
        new rows in its own dtype.  terms ((d1, w1), (d2, w2)) in place of delta: the addend is w1 d1 + w2 d2."""
        T, H = residual.shape
        delta2, w1, w2 = None, 1.0, 0.0
        if terms is not None:
            (delta, w1), (delta2, w2) = terms
            if delta2.dtype != delta.dtype or delta2.shape != delta.shape:
                raise ShapeError("postnorm_scale_add: two addends of one shape and dtype")
        if residual.dtype != torch.float32 or (delta is not None and tuple(delta.shape) != (T, H)) or \
                (out is not None and tuple(out.shape) != (T, H)):
            raise ShapeError(f"postnorm_scale_add: residual {tuple(residual.shape)} {residual.dtype}")
        self._check(self.lib.srlm_postnorm_scale_add(
            _ptr(residual), _ptr(delta), _ptr(delta2), C.c_float(w1), C.c_float(w2),
            dtype_code(delta.dtype) if delta is not None else 0, _ptr(weight), C.c_float(alpha),
            C.c_float(eps), C.c_int(int(unit_offset)), _ptr(out), dtype_code(out.dtype) if out is not None else 0,
            C.c_int(T), C.c_int(H), _stream()), "postnorm_scale_add")

    def rmsnorm_columns(self, x, column, width, weight, eps, out, unit_offset=False):
        """out [T, width] = RMS norm over the columns [column, column + width) of x (float32, row-major), times weight
        (float32 [width]; None: no weight)."""
        ptr, ld = self._columns(x, column, width)
        self._check(self.lib.srlm_rmsnorm_columns(ptr, ld, _ptr(weight), C.c_float(eps), C.c_int(int(unit_offset)), _ptr(out),
                                                  dtype_code(out.dtype), C.c_int(x.shape[0]), C.c_int(width), _stream()),
                    "rmsnorm_columns")

    ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1}

    def activation(self, x, out, kind, bias=None, column=0):
        """out [T, F] = act(x[:, column : column + F] + bias); kind "gelu" (exact) or "gelu_tanh"."""
        T, F = out.shape
        if not x.is_cuda or x.stride(1) != 1 or x.shape[1] < column + F:
            raise ShapeError("activation: columns of a row-major CUDA tensor are wanted")
        self._check(self.lib.srlm_activation(C.c_void_p(x.data_ptr() + x.element_size() * column), dtype_code(x.dtype),
                                             C.c_longlong(x.stride(0)), _ptr(bias), _ptr(out), dtype_code(out.dtype),
                                             C.c_int(T), C.c_int(F), C.c_int(self.ACTIVATIONS[kind]), _stream()), "activation")

    def weighted_sum(self, a, wa, b, wb, out):
        """out = wa * a + wb * b (a and b of one dtype, float32 sums)."""
        if a.shape != b.shape or a.dtype != b.dtype or out.shape != a.shape:
            raise ShapeError("weighted_sum: operands of one shape and dtype")
        self._check(self.lib.srlm_weighted_sum(_ptr(a), C.c_float(wa), _ptr(b), C.c_float(wb), dtype_code(a.dtype),
                                               _ptr(out), dtype_code(out.dtype), C.c_longlong(a.numel()), _stream()),
                    "weighted_sum")

    # ---- short convolutions over time ---------------------------------------------------------------
    def short_conv(self, ctx, x, column, channels, weight, state, state_off, out, in_bias=None, out_bias=None, out_low=None):
        """out float32 [T, channels] = the causal convolution over time of the columns [column, + channels) of x (float32),
        per channel with weight float32 [channels, taps]; in_bias is added to every input, out_bias to every result.  A
        portion's first tokens read the slot's carried inputs ([taps - 1][channels] floats at state_off of its row of
        ``state``, float32 [slots, row]); ``conv_carry`` renews them afterwards.  out_low: a copy in its own dtype."""
        ptr, ld = self._columns(x, column, channels)
        self._check(self.lib.srlm_short_conv(
            ptr, ld, _ptr(in_bias), _ptr(weight), _ptr(out_bias), _ptr(state), C.c_longlong(state.stride(0)),
            C.c_int(state_off), _ptr(ctx.entry_of_token), _ptr(ctx.cu_q), _ptr(ctx.slots), _ptr(out), _ptr(out_low),
            dtype_code(out_low.dtype) if out_low is not None else 0, C.c_int(x.shape[0]), C.c_int(channels),
            C.c_int(weight.shape[1]), _stream()), "short_conv")

    def conv_carry(self, ctx, x, column, channels, taps, state, state_off, in_bias=None):
        """The slots' carried inputs of a short convolution <- the last taps - 1 inputs of every entry (what was carried
        before counts as the inputs ahead of the portion)."""
        if taps <= 1:
            return
        ptr, ld = self._columns(x, column, channels)
        self._check(self.lib.srlm_conv_carry(ptr, ld, _ptr(in_bias), _ptr(state), C.c_longlong(state.stride(0)),
                                             C.c_int(state_off), _ptr(ctx.cu_q), _ptr(ctx.slots), C.c_int(ctx.n_entries),
                                             C.c_int(channels), C.c_int(taps), _stream()), "conv_carry")

    def conv_norm_rope_append(self, ctx, proj, conv_w, state, state_off, q_norm_w, k_norm_w, eps, rotation, q_out, k_cache,
                              v_cache, kv_slot, nq, nkv, dk, dv):
        """From a stacked q | k | v projection (float32 [T, >= nq dk + nkv (dk + dv)]): every channel through its short
        convolution (conv_w float32 [channels, taps], the slots' carried inputs in ``state``), every q and k head
        RMS-normed with q_norm_w / k_norm_w (float32 [dk]; None: not normed) and its leading pairs turned; q to q_out
        (float32 or bfloat16), k and v to the pages."""
        pairs = rotation.pairs if rotation is not None else 0
        self._check(self.lib.srlm_conv_norm_rope_append(
            _ptr(proj), C.c_longlong(proj.stride(0)), _ptr(conv_w), _ptr(state), C.c_longlong(state.stride(0)),
            C.c_int(state_off), _ptr(q_norm_w), _ptr(k_norm_w), C.c_float(eps or 0.0),
            _ptr(rotation.cos if pairs else None), _ptr(rotation.sin if pairs else None), C.c_int(pairs),
            C.c_int(int(bool(pairs and rotation.interleaved))), _ptr(ctx.entry_of_token), _ptr(ctx.cu_q), _ptr(ctx.slots),
            _ptr(kv_slot), _ptr(q_out), dtype_code(q_out.dtype), _ptr(k_cache), _ptr(v_cache), dtype_code(k_cache.dtype),
            C.c_int(proj.shape[0]), C.c_int(nq), C.c_int(nkv), C.c_int(dk), C.c_int(dv), C.c_int(k_cache.shape[2]),
            C.c_int(conv_w.shape[1]), _stream()), "conv_norm_rope_append")

    # ---- the matrix memory ----------------------------------------------------------------------------
    def matrix_memory_recurrence(self, ctx, proj, bias_i, bias_f, cap, floor, state, o_out, H, d, dv):
        """o_out float32 [T, H dv]: the read-outs of a matrix memory with exponential gates, token by token, from the
        stacked projection q | k | v | output gate | i | f (float32); state float32 [slots, H dv d + H d + H]
        (S of a head with the rows of a value column contiguous, then n, then m)."""
        self._check(self.lib.srlm_matrix_memory_recurrence(
            _ptr(proj), C.c_longlong(proj.stride(0)), _ptr(bias_i), _ptr(bias_f), C.c_float(cap), C.c_float(floor),
            _ptr(state), C.c_longlong(state.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.slots), _ptr(o_out),
            C.c_int(ctx.n_entries), C.c_int(ctx.max_q_len), C.c_int(H), C.c_int(d), C.c_int(dv), _stream()),
            "matrix_memory_recurrence")

    def matrix_memory_output(self, o, norm_w, eps, proj, g_off, out, H, dv):
        """out [T, H dv] = per head o / sqrt(mean(o^2) + eps), times norm_w (float32 [H dv]), times the logistic of the
        columns g_off .. of proj."""
        self._check(self.lib.srlm_matrix_memory_output(
            _ptr(o), _ptr(norm_w), C.c_float(eps), _ptr(proj), C.c_longlong(proj.stride(0)), C.c_int(g_off), _ptr(out),
            dtype_code(out.dtype), C.c_int(o.shape[0]), C.c_int(H), C.c_int(dv), _stream()), "matrix_memory_output")

    # ---- the gated linear recurrence --------------------------------------------------------------------
    def recurrence_gates(self, u, Ra, Ri, ba, bi, rate, a_out, b_out, blocks):
        """a_out = exp(-rate * logistic(Ra u + ba)), b_out = sqrt(1 - a^2) * logistic(Ri u + bi) * u; u float32 [T, C];
        Ra, Ri [blocks, C / blocks, C / blocks] (block-diagonal, [out, in])."""
        T, Cn = u.shape
        self._check(self.lib.srlm_recurrence_gates(_ptr(u), _ptr(Ra), _ptr(Ri), dtype_code(Ra.dtype), _ptr(ba), _ptr(bi),
                                                   _ptr(rate), _ptr(a_out), _ptr(b_out), C.c_int(T), C.c_int(Cn),
                                                   C.c_int(blocks), _stream()), "recurrence_gates")

    def linear_recurrence(self, ctx, a, b, y, y_column, y_bias, state, out, in_segments=False):
        """S <- a S + b per channel and token, from the slots' S (the first C floats of a row of ``state``), renewed at
        the end; out [T, C] = S * gelu_tanh(y[:, y_column : + C] + y_bias).  in_segments: every entry's tokens in 32
        segments walked side by side (for long portions; the sums are formed in another order)."""
        T, Cn = a.shape
        ptr, ld = self._columns(y, y_column, Cn)
        self._check(self.lib.srlm_linear_recurrence(_ptr(a), _ptr(b), ptr, ld, _ptr(y_bias), _ptr(state),
                                                    C.c_longlong(state.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.slots),
                                                    _ptr(out), dtype_code(out.dtype), C.c_int(ctx.n_entries), C.c_int(Cn),
                                                    C.c_int(int(in_segments)), _stream()), "linear_recurrence")

    # ---- attention over a cached latent ----------------------------------------------------
    def latent_append(self, proj, c_off, norm_w, eps, rotation, cache, kv_slot, rank, rot, q_norm=None):
        """cache row of each token = [rms_norm(proj[c_off : c_off + rank]) * norm_w | rotated proj[.. + rot]].
        q_norm (column, width, weight, out): the same kernel also writes out [T, width] = rms_norm(proj[column : column +
        width]) * weight (a latent of the queries that the same stacked projection holds)."""
        pairs = rotation.pairs if rotation is not None else 0
        q_col, q_width, q_w, q_out = q_norm if q_norm is not None else (0, 0, None, None)
        self._check(self.lib.srlm_latent_append(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), C.c_int(c_off), _ptr(norm_w),
            C.c_float(eps), _ptr(rotation.cos if pairs else None), _ptr(rotation.sin if pairs else None),
            C.c_int(pairs), C.c_int(int(bool(pairs and not rotation.interleaved))), _ptr(cache), dtype_code(cache.dtype),
            _ptr(kv_slot), C.c_int(proj.shape[0]), C.c_int(rank), C.c_int(rot), C.c_int(q_col), C.c_int(q_width),
            _ptr(q_w), _ptr(q_out), dtype_code(q_out.dtype) if q_out is not None else 0, _stream()), "latent_append")

    def latent_absorb(self, proj, uk, rotation, q_out, heads, dim, rot, rank):
        """q_out float32 [T, heads, rank + rot] = per head [uk_h^T q_h | rotated rest of the head]; uk [heads, dim, rank]."""
        pairs = rotation.pairs if rotation is not None else 0
        self._check(self.lib.srlm_latent_absorb(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), _ptr(uk), dtype_code(uk.dtype),
            _ptr(rotation.cos if pairs else None), _ptr(rotation.sin if pairs else None), C.c_int(pairs),
            C.c_int(int(bool(pairs and not rotation.interleaved))), _ptr(q_out),
            C.c_int(proj.shape[0]), C.c_int(heads), C.c_int(dim), C.c_int(rot), C.c_int(rank), _stream()),
            "latent_absorb")

    def latent_expand(self, o_lat, uv_t, proj, g_off, out, heads, rank, dv):
        """out [T, heads * dv] = per head (uv_t_h^T o_lat_h) * sigmoid(proj[:, g_off + h]); uv_t [heads, rank, dv];
        g_off < 0: no gate."""
        self._check(self.lib.srlm_latent_expand(
            _ptr(o_lat), _ptr(uv_t), dtype_code(uv_t.dtype), _ptr(proj), dtype_code(proj.dtype),
            C.c_longlong(proj.stride(0)), C.c_int(g_off), _ptr(out), dtype_code(out.dtype), C.c_int(o_lat.shape[0]),
            C.c_int(heads), C.c_int(rank), C.c_int(dv), _stream()), "latent_expand")

    def latent_prompt_takes(self, dim, rot, dv, rank) -> bool:
        """Whether prompts of a latent attention of these sizes may attend in the heads' own space on tensor cores."""
        return bool(self.latent_prompts_in_head_space and self.general_attention_on_tensor_cores
                    and self.lib.srlm_latent_prefill_attention_takes(C.c_int(dim), C.c_int(rot), C.c_int(dv), C.c_int(rank)))

    def latent_gather(self, ctx, cache, dst, block_table, cu_kv, rank, kv_first=None):
        """dst[cu_kv[e] + j] = the latent (first ``rank`` elements of the page row) of key j of entry e, for j from
        kv_first[e] (None: 0) on; zeros where the page has been given back."""
        self._check(self.lib.srlm_latent_gather(
            _ptr(cache), dtype_code(cache.dtype), _ptr(dst), _ptr(block_table), C.c_int(block_table.stride(0)),
            _ptr(cu_kv), _ptr(kv_first), _ptr(ctx.kv_lens), C.c_int(ctx.n_entries), C.c_int(ctx.max_kv_len),
            C.c_int(cache.shape[2]), C.c_int(cache.shape[3]), C.c_int(rank), _stream()), "latent_gather")

    def latent_rotate_q(self, proj, rotation, q_out, heads, dim, rot):
        pairs = rotation.pairs if rotation is not None else 0
        self._check(self.lib.srlm_latent_rotate_q(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), _ptr(rotation.cos if pairs else None),
            _ptr(rotation.sin if pairs else None), C.c_int(pairs), C.c_int(int(bool(pairs and not rotation.interleaved))),
            _ptr(q_out), C.c_int(proj.shape[0]), C.c_int(heads), C.c_int(dim), C.c_int(rot), _stream()), "latent_rotate_q")

    def latent_prefill_attention(self, ctx, q, pages, kv_rows, cu_kv, out, block_table, heads, dim, rot, dv, rank,
                                 v_off, scale, window=0):
        """Causal attention of prompts in the heads' own space: q float32 [T, heads * (dim + rot)]; kv_rows bfloat16
        [keys of all entries, >= v_off + heads * dv] with the heads' unrotated keys and, from column v_off, values;
        the rotated key part comes from the pages."""
        self._check(self.lib.srlm_latent_prefill_attention(
            _ptr(q), _ptr(pages), _ptr(kv_rows), C.c_longlong(kv_rows.stride(0)), _ptr(cu_kv), _ptr(out),
            dtype_code(out.dtype), _ptr(block_table), C.c_int(block_table.stride(0)), _ptr(ctx.cu_q), _ptr(ctx.kv_lens),
            C.c_int(ctx.n_entries), C.c_int(ctx.max_q_len), C.c_int(heads), C.c_int(dim), C.c_int(rot), C.c_int(dv),
            C.c_int(rank), C.c_int(v_off), C.c_int(pages.shape[2]), C.c_float(scale), C.c_int(window or 0), _stream()),
            "latent_prefill_attention")

    def head_gate(self, x, proj, g_off, out, heads, dv):
        """out[t, h, :] = x[t, h, :] * sigmoid(proj[t, g_off + h]); x float32, or bfloat16 (out may then be x itself);
        g_off < 0: no gate."""
        self._check(self.lib.srlm_head_gate(
            _ptr(x), dtype_code(x.dtype), _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), C.c_int(g_off), _ptr(out),
            dtype_code(out.dtype), C.c_int(x.shape[0]), C.c_int(heads), C.c_int(dv), _stream()), "head_gate")

    # ---- the gated delta rule ------------------------------------------------------------------
    def delta_prepare(self, ctx, proj, conv_w, a_log, dt_bias, state, qkv_out, beta_out, decay_out, qk_out, H, G, dk,
                      dv, taps, unit_eps):
        """Convolution + SiLU of the q | k | v columns of proj (carrying each slot's last taps-1 inputs in its
        state), unit vectors, beta, decay and q . k (float32 [T, G]) for every token; then the slots' carried inputs are renewed.
        state: float32 [slots, state_size], laid out as csrc/kernels/delta_rule.cu says."""
        self._check(self.lib.srlm_delta_prepare(
            _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)), _ptr(conv_w), _ptr(a_log), _ptr(dt_bias),
            _ptr(state), C.c_longlong(state.stride(0)), _ptr(ctx.entry_of_token), _ptr(ctx.cu_q), _ptr(ctx.slots),
            C.c_int(ctx.n_entries), _ptr(qkv_out), _ptr(beta_out), _ptr(decay_out), _ptr(qk_out), C.c_int(proj.shape[0]),
            C.c_int(H), C.c_int(G), C.c_int(dk), C.c_int(dv), C.c_int(taps), C.c_float(unit_eps), _stream()), "delta_prepare")
        if taps > 1:
            self.launches += 1

    def delta_recurrence(self, ctx, qkv, beta, decay, qk, state, o_out, H, G, dk, dv):
        self._check(self.lib.srlm_delta_recurrence(
            _ptr(qkv), _ptr(beta), _ptr(decay), _ptr(qk), _ptr(state), C.c_longlong(state.stride(0)), _ptr(ctx.cu_q),
            _ptr(ctx.slots), C.c_int(ctx.n_entries), _ptr(o_out), C.c_int(H), C.c_int(G), C.c_int(dk), C.c_int(dv),
            _stream()), "delta_recurrence")

    def delta_output(self, o, norm_w, eps, proj, gate_off, out, H, dv):
        self._check(self.lib.srlm_delta_output(
            _ptr(o), _ptr(norm_w), C.c_float(eps), _ptr(proj), dtype_code(proj.dtype), C.c_longlong(proj.stride(0)),
            C.c_int(gate_off), _ptr(out), dtype_code(out.dtype), C.c_int(o.shape[0]), C.c_int(H), C.c_int(dv),
            _stream()), "delta_output")

    # ---- sampling -------------------------------------------------------------
    def argmax(self, logits, out_tokens, bad_flag):
        n, V = logits.shape
        self._check(self.lib.srlm_argmax(_ptr(logits), C.c_longlong(logits.stride(0)), C.c_int(n), C.c_int(V),
                                         _ptr(out_tokens), _ptr(bad_flag), _stream()), "argmax")

    def sample(self, logits, temperature, top_k, top_p, penalty, uniform, history, hist_offsets, out_tokens,
               bad_flag, scratch):
        """scratch: float32 [n, V] that the kernel may overwrite (the adjusted values of each row)."""
        n, V = logits.shape
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < n * V:
            raise ShapeError("sample: scratch must hold n x V float32 values")
        self._check(self.lib.srlm_sample(_ptr(logits), C.c_longlong(logits.stride(0)), C.c_int(n), C.c_int(V),
                                         _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(penalty),
                                         _ptr(uniform), _ptr(history), _ptr(hist_offsets), _ptr(scratch),
                                         _ptr(out_tokens), _ptr(bad_flag), _stream()), "sample")


ops = KernelLibrary()
