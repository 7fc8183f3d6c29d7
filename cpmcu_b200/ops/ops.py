"""The kernel library as Python calls, bound to one compute dtype.

``Ops(torch.bfloat16)`` is the serving path: bf16 activations, weights and cache,
fp32 residual stream, norms, softmax and logits.  ``Ops(torch.float32)`` is the
true 32-bit path: every tensor fp32 and every matrix product done by this
library's own fp32 FMA kernel, never by a library routine that may pick a
reduced-precision mode.

Matrix products of the bf16 path go to cuBLAS through torch, as the reference's
do through ``cublasGemmEx`` (src/model/linear.cuh:8-37), unless a hand-written
kernel of this library takes the shape.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import library
from .library import check

from ..parts.base import PAGE_TOKENS, QUERY_TILE_TOKENS

F32, BF16 = 0, 1
FAST_HEAD_DIMS = (32, 64, 96, 128)       # head sizes the tensor-core attention kernels are built for
PREFILL_TILE_ROWS = QUERY_TILE_TOKENS    # query tokens per block of the prefill attention kernel


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _current_stream() -> int:
    """Handle of the stream torch would launch on now (the raw query is an order of magnitude cheaper than
    building a Stream object for every kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class Ops:
    def __init__(self, dtype: torch.dtype, device: "torch.device | str" = "cuda:0"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.dtype = dtype
        self.code = F32 if dtype == torch.float32 else BF16
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise library.KernelLibraryError("this library runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise library.KernelLibraryError("no CUDA device is available; there is no CPU path")
        self.lib = library.load()
        if int(self.lib.cpm_page_tokens()) != PAGE_TOKENS or int(self.lib.cpm_prefill_attention_tile_rows()) != PREFILL_TILE_ROWS:
            raise library.KernelLibraryError("the kernel library was built for another page or query-tile size than the package")
        self.element_size = 4 if dtype == torch.float32 else 2
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.use_tcgen05 = os.environ.get("CPMCU_TCGEN05", "1") != "0"
        self.use_tcgen05_attention = os.environ.get("CPMCU_TCGEN05_ATTENTION", "1") != "0"
        self.use_tcgen05_sink = os.environ.get("CPMCU_TCGEN05_SINK", "1") != "0"                # sink window attention of prompts
        self.use_tcgen05_listed = os.environ.get("CPMCU_TCGEN05_LISTED", "1") != "0"      # block-list attention of prompts
        self.tcgen05_pair = os.environ.get("CPMCU_TCGEN05_PAIR", "0") == "1"      # pairs of blocks on 256-row tiles
        self.workspace = None       # cpmcu_b200.memory.Workspace: where a step's intermediates live (None: torch's allocator)
        self.weights = None         # cpmcu_b200.memory.Region that holds the weights (None: torch's allocator)

    _stream = staticmethod(_current_stream)

    # ---- checks ----
    def _act(self, t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous {self.dtype} CUDA tensor, got {t.dtype} "
                             f"{'cuda' if t.is_cuda else 'cpu'} contiguous={t.is_contiguous()}")
        return t

    @staticmethod
    def _i32(t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous int32 CUDA tensor")
        return t

    @staticmethod
    def _f32(t: torch.Tensor, what: str) -> torch.Tensor:
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{what}: needs a contiguous float32 CUDA tensor")
        return t

    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A tensor for an intermediate of the step: from the workspace when one is attached (it is valid until the
        workspace reuses its place, at the latest when the next step begins), else from torch's allocator."""
        if self.workspace is not None:
            return self.workspace.alloc(shape, dtype or self.dtype)
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def result(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """A tensor the step hands to its caller (logits, sampled tokens): never from the workspace, so that it
        stays valid after later steps."""
        return torch.empty(*shape, dtype=dtype or self.dtype, device=self.device)

    def keep(self, t: torch.Tensor) -> torch.Tensor:
        """A weight for good: copied into the arena's weight region when one is attached (the copy replaces the
        tensor the loader made), else the tensor itself."""
        if self.weights is None or t.device.type == "meta":
            return t
        own = self.weights.tensor(t.shape, t.dtype, what="weights")
        own.copy_(t)
        return own

    # ---- the workspace's lifetimes (no-ops without a workspace) ----
    def begin_step(self) -> None:
        if self.workspace is not None:
            self.workspace.begin_step()

    def begin_layer(self, k: int) -> None:
        if self.workspace is not None:
            self.workspace.begin_layer(k)

    def end_layers(self) -> None:
        if self.workspace is not None:
            self.workspace.end_layers()

    # ---- rows ----
    def embed(self, ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
        """ids int32 [tokens], table [vocab, hidden] -> fp32 [tokens, hidden] = table[ids] * scale."""
        self._i32(ids, "embed ids")
        self._act(table, "embedding table")
        n, hidden = ids.numel(), table.shape[1]
        out = self.empty(n, hidden, dtype=torch.float32)
        check(self.lib.cpm_embed_rows(_ptr(ids), _ptr(table), _ptr(out), n, hidden, float(scale), self.code,
                                      self._stream()), "embed")
        return out

    def add_rmsnorm(self, x: torch.Tensor, delta: Optional[torch.Tensor], alpha: float, weight: torch.Tensor,
                    eps: float, rows: Optional[torch.Tensor] = None, delta2: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x fp32 [tokens, hidden] (+= alpha*delta, and + alpha*delta2 when a second addend is given; written back when
        rows is None) -> normed rows."""
        self._f32(x, "residual stream")
        hidden = x.shape[-1]
        if delta is not None:
            self._act(delta, "residual addend")
            if delta.shape != x.shape:
                raise ValueError(f"residual addend {tuple(delta.shape)} does not match the stream {tuple(x.shape)}")
        if delta2 is not None:
            self._act(delta2, "second residual addend")
            if delta is None or delta2.shape != x.shape:
                raise ValueError("a second residual addend goes with a first one of the stream's shape")
        if weight.dtype not in (torch.float32, self.dtype) or weight.numel() != hidden or weight.device.type != self.device.type:
            raise ValueError("norm weight: needs [hidden] in float32 or the compute dtype")
        n_rows = x.shape[0] if rows is None else rows.numel()
        if rows is not None:
            self._i32(rows, "norm rows")
        y = self.empty(n_rows, hidden)
        check(self.lib.cpm_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(delta2), float(alpha), _ptr(weight),
                                       1 if weight.dtype == torch.float32 else 0, _ptr(y), _ptr(rows), n_rows,
                                       hidden, float(eps), 1 if rows is None else 0, self.code, self._stream()),
              f"rmsnorm (hidden {hidden})")
        return y

    def residual_add(self, x: torch.Tensor, delta: torch.Tensor, alpha: float) -> None:
        self._f32(x, "residual stream")
        self._act(delta, "residual addend")
        if delta.shape != x.shape:
            raise ValueError("residual addend does not match the stream")
        check(self.lib.cpm_residual_add(_ptr(x), _ptr(delta), float(alpha), x.numel(), self.code, self._stream()),
              "residual add")

    def silu_mul(self, gu: torch.Tensor, interleave: int = 0) -> torch.Tensor:
        """gu [tokens, 2*inter] -> silu(gate) * up, [tokens, inter].  interleave 0: rows are
        [gate | up]; 8: blocks of 8 gate values followed by the 8 up values of the same features."""
        self._act(gu, "gate_up")
        n, two_i = gu.shape
        h = self.empty(n, two_i // 2)
        check(self.lib.cpm_silu_mul(_ptr(gu), _ptr(h), n, two_i // 2, interleave, self.code, self._stream()), "silu_mul")
        return h

    # ---- layer norm, token shift, additions to the stream ----
    def embed_sinusoid(self, ids: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, freq: torch.Tensor,
                       scale: float) -> torch.Tensor:
        """fp32 [tokens, hidden] = table[ids] * scale + (sin | cos)(positions * freq), even entries sin, odd cos."""
        self._i32(ids, "embed ids")
        self._i32(positions, "positions")
        self._act(table, "embedding table")
        self._f32(freq, "frequencies")
        n, hidden = ids.numel(), table.shape[1]
        if freq.numel() * 2 != hidden:
            raise ValueError("sinusoidal embedding: needs hidden/2 frequencies")
        out = self.empty(n, hidden, dtype=torch.float32)
        check(self.lib.cpm_embed_sinusoid(_ptr(ids), _ptr(positions), _ptr(table), _ptr(freq), _ptr(out), n, hidden,
                                          float(scale), self.code, self._stream()), "embed_sinusoid")
        return out

    def layernorm(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float,
                  rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 stream [tokens, hidden] -> (x - mean) / sqrt(var + eps) * w + b of all or of the listed rows."""
        self._f32(x, "residual stream")
        self._f32(w, "norm weight")
        self._f32(b, "norm bias")
        hidden = x.shape[-1]
        n_rows = x.shape[0] if rows is None else rows.numel()
        if rows is not None:
            self._i32(rows, "norm rows")
        y = self.empty(n_rows, hidden)
        check(self.lib.cpm_layernorm_rows(_ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(rows), n_rows, hidden, float(eps),
                                          self.code, self._stream()), f"layernorm (hidden {hidden})")
        return y

    def layernorm_shift(self, ctx, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, mix: torch.Tensor,
                        state: torch.Tensor) -> torch.Tensor:
        """h = layernorm(x); y_t = h_t + (h_{t-1} - h_t) * mix, with ``state`` [slots, hidden] fp32 giving the h before
        a sequence's first token of the step and taking the h of its last."""
        self._f32(x, "residual stream")
        self._f32(state, "shift state")
        for t, what in ((w, "norm weight"), (b, "norm bias"), (mix, "shift vector")):
            self._f32(t, what)
        n, hidden = x.shape
        if state.shape[-1] != hidden:
            raise ValueError("shift state does not match the hidden size")
        y = self.empty(n, hidden)
        check(self.lib.cpm_layernorm_shift(_ptr(x), _ptr(w), _ptr(b), _ptr(mix), _ptr(state), _ptr(ctx.positions),
                                           _ptr(ctx.token_seq), _ptr(ctx.cu_q), _ptr(ctx.slot_dev), _ptr(y), n, hidden,
                                           float(eps), self.code, self._stream()), f"layernorm_shift (hidden {hidden})")
        return y

    def post_norm_add(self, x: torch.Tensor, a: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float,
                      then=None) -> Optional[torch.Tensor]:
        """x += layernorm(a) with (w, b); ``then`` = (w2, b2): also returns layernorm(x) with those."""
        self._f32(x, "residual stream")
        self._act(a, "sublayer output")
        if a.shape != x.shape:
            raise ValueError(f"sublayer output {tuple(a.shape)} does not match the stream {tuple(x.shape)}")
        n, hidden = x.shape
        y = self.empty(n, hidden) if then is not None else None
        w2, b2 = then if then is not None else (None, None)
        check(self.lib.cpm_post_norm_add(_ptr(x), _ptr(a), _ptr(w), _ptr(b), _ptr(w2), _ptr(b2), _ptr(y), n, hidden,
                                         float(eps), self.code, self._stream()), f"post_norm_add (hidden {hidden})")
        return y

    def stream_inject(self, x: torch.Tensor, saved: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> None:
        """x += saved (same shape, fp32) + vec (one value per column, fp32); either may be None."""
        self._f32(x, "residual stream")
        if saved is not None and saved.shape != x.shape:
            raise ValueError("saved stream does not match the stream")
        if vec is not None and vec.numel() != x.shape[-1]:
            raise ValueError("vector does not match the hidden size")
        check(self.lib.cpm_stream_inject(_ptr(x), _ptr(saved), _ptr(vec), x.shape[0], x.shape[1], self._stream()),
              "stream_inject")

    # ---- recurrence ----
    MINGRU_TILE_MIN_TOKENS = 32      # from this many tokens in a sequence on, a prompt's recurrence runs tile-parallel

    def mingru_scan(self, ctx, proj: torch.Tensor, bz: torch.Tensor, bx: torch.Tensor, state: torch.Tensor,
                    width: int) -> torch.Tensor:
        """proj fp32 [tokens, 3*width] = [z | x | g] raw projections -> S_t * silu(g_t) [tokens, width], with the
        per-sequence ``state`` [slots, width] fp32 read at a sequence's first token and written at its last."""
        self._f32(proj, "recurrence projections")
        self._f32(state, "recurrence state")
        n = proj.shape[0]
        if proj.shape[1] != 3 * width or state.shape[-1] != width:
            raise ValueError("recurrence: projections must be [tokens, 3*width] and the state [slots, width]")
        out = self.empty(n, width)
        tiles = ctx.q_tiles
        if ctx.is_decode or tiles is None or ctx.max_q_len < self.MINGRU_TILE_MIN_TOKENS:
            check(self.lib.cpm_mingru_scan(_ptr(proj), _ptr(bz), _ptr(bx), _ptr(state), _ptr(ctx.positions), _ptr(ctx.cu_q),
                                           _ptr(ctx.slot_dev), None, None, 0, 0, None, _ptr(out), ctx.n_seqs, width,
                                           self.code, self._stream()), "mingru_scan")
            return out
        tile_seq, tile_row, n_tiles = tiles
        summary = self.empty(int(self.lib.cpm_mingru_summary_floats(n_tiles, width)), dtype=torch.float32)
        check(self.lib.cpm_mingru_scan(_ptr(proj), _ptr(bz), _ptr(bx), _ptr(state), _ptr(ctx.positions), _ptr(ctx.cu_q),
                                       _ptr(ctx.slot_dev), _ptr(tile_seq), _ptr(tile_row), n_tiles, QUERY_TILE_TOKENS,
                                       _ptr(summary), _ptr(out), ctx.n_seqs, width, self.code, self._stream()),
              "mingru_scan (tiles)")
        LAUNCHES_EXTRA[0] += 1
        return out

    # ---- attention over cached latents ----
    def latent_norm_store(self, ctx, proj: torch.Tensor, g_q: torch.Tensor, g_kv: torch.Tensor, lane, q_rank: int,
                          rank: int, eps: float, write_cache: bool = True, rot_dim: int = 0,
                          inv_freq: Optional[torch.Tensor] = None, adjacent: bool = False) -> torch.Tensor:
        """proj fp32 rows that begin [q_rank | rank | rot_dim]: RMS-norms the first two parts; returns the query latent
        [tokens, q_rank] and stores the key-value latent into the lane's pages at each token's position, followed (with
        ``rot_dim``) by the third part turned by the position: pairs (i, i + rot_dim/2), or (2i, 2i + 1) with ``adjacent``,
        angle position * inv_freq[i].  A cache row is [rank + rot_dim]."""
        self._f32(proj, "latent projections")
        n = proj.shape[0]
        if proj.shape[1] < q_rank + rank + rot_dim:
            raise ValueError("latent projections must be [tokens, >= q_rank + rank + rot_dim]")
        if rot_dim:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != rot_dim // 2:
                raise ValueError("inv_freq needs rot_dim/2 entries")
        if write_cache and lane.k.shape[-1] != rank + rot_dim:
            raise ValueError(f"latent_norm_store: the lane's rows hold {lane.k.shape[-1]} values, not {rank + rot_dim}")
        cq = self.empty(n, q_rank)
        cache = lane.k if write_cache else None
        check(self.lib.cpm_latent_norm_store(_ptr(proj), proj.stride(0), _ptr(g_q), _ptr(g_kv), _ptr(cq), _ptr(cache),
                                             _ptr(ctx.positions), _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                             lane.page_table.shape[1], n, q_rank, rank, int(rot_dim),
                                             _ptr(inv_freq) if rot_dim else None, 1 if adjacent else 0, float(eps), self.code,
                                             self._stream()), "latent_norm_store")
        return cq

    def rotate_heads(self, ctx, x: torch.Tensor, n_heads: int, first: int, rot_dim: int, inv_freq: torch.Tensor,
                     adjacent: bool = False) -> torch.Tensor:
        """x fp32 [tokens, heads * dh] -> [tokens, heads * dh] in the compute dtype with the channels [first, first +
        rot_dim) of every head turned by the token's position (pairs as in ``latent_norm_store``)."""
        self._f32(x, "heads to rotate")
        self._f32(inv_freq, "inv_freq")
        n, dh = x.shape[0], x.shape[1] // n_heads
        out = self.empty(n, n_heads * dh)
        check(self.lib.cpm_rotate_heads(_ptr(x), _ptr(out), _ptr(ctx.positions), _ptr(inv_freq), n, n_heads, dh, int(first),
                                        int(rot_dim), 1 if adjacent else 0, self.code, self._stream()), "rotate_heads")
        return out

    def head_gate(self, x: torch.Tensor, gate: torch.Tensor, n_heads: int) -> torch.Tensor:
        """In place: x [tokens, heads * dv] (compute dtype) times sigmoid(gate [tokens, heads]) head by head; the gate is
        fp32 and may be a slice of wider rows."""
        self._act(x, "heads to gate")
        n = x.shape[0]
        if gate.dtype != torch.float32 or gate.shape != (n, n_heads) or gate.stride(1) != 1:
            raise ValueError("head_gate: the gate must be fp32 [tokens, heads]")
        check(self.lib.cpm_head_gate(_ptr(x), _ptr(gate), gate.stride(0), n, n_heads, x.numel() // (n * n_heads), self.code,
                                     self._stream()), "head_gate")
        return x

    HEAD_PROJECT_LIBRARY_MIN_TOKENS = 64      # from this many tokens on, the per-head maps of the bf16 path are batched library products

    def head_project_by_library(self, n_tokens: int) -> bool:
        return self.code == BF16 and n_tokens >= self.HEAD_PROJECT_LIBRARY_MIN_TOKENS

    def head_project(self, x: torch.Tensor, w: torch.Tensor, n_heads: int, out_f32: bool) -> torch.Tensor:
        """x [tokens, heads * k] (or [tokens, heads, k]; fp32 or the compute dtype) times w [heads, k, n] head by
        head -> [tokens, heads, n], fp32 or the compute dtype.  Many tokens of bf16 input go to the library's batched
        product (one product per head over strided views), few tokens and the 32-bit path to this library's kernel."""
        self._act(w, "per-head matrices")
        n_tok = x.shape[0]
        H, K, N = w.shape
        if H != n_heads or x.numel() != n_tok * H * K or not x.is_contiguous():
            raise ValueError(f"head_project: input {tuple(x.shape)} against matrices {tuple(w.shape)}")
        in_f32 = x.dtype == torch.float32
        if not in_f32 and x.dtype != self.dtype:
            raise ValueError("head_project: the input must be fp32 or the compute dtype")
        out = self.empty(n_tok, H, N, dtype=torch.float32 if out_f32 else self.dtype)
        if self.head_project_by_library(n_tok) and not in_f32:
            by_head = torch.bmm(x.view(n_tok, H, K).transpose(0, 1), w, out_dtype=out.dtype) if out_f32 else \
                torch.bmm(x.view(n_tok, H, K).transpose(0, 1), w)
            out.copy_(by_head.transpose(0, 1))
            return out
        check(self.lib.cpm_head_project(_ptr(x), _ptr(w), _ptr(out), n_tok, H, K, N, 1 if in_f32 else 0,
                                        1 if out_f32 else 0, self.code, self._stream()), f"head_project ({K} -> {N})")
        return out

    LATENT_MAX_SPLITS = 32      # most blocks that share the keys of one token and head group

    def latent_attention_splits(self, ctx, n_tokens: int, n_heads: int, window: int) -> int:
        """How many blocks share the keys of one token and head group in the tensor-core kernel: one, unless the step's
        tokens leave most SMs idle (a decode step) and there are enough keys.  A block walks its tiles of 32 keys one
        after the other, each a round trip to L2, so a decode step aims at three blocks per SM with at least two tiles
        each (a step of batch 8 at the 4,096-wide sizes: 44 us a launch with 9 shares, the device's time)."""
        blocks = n_tokens * ((n_heads + 15) // 16)
        if blocks * 2 > self.sm_count:
            return 1
        keys = min(window, ctx.max_kv_len) if window else ctx.max_kv_len      # in a recorded step an upper bound
        return max(1, min(self.LATENT_MAX_SPLITS, 3 * self.sm_count // blocks, ((keys + 31) // 32) // 2))

    def latent_attention_on_tensor_cores(self, rank: int) -> bool:
        return self.code == BF16 and rank % 16 == 0 and rank <= 512

    def latent_attention(self, ctx, q_lat: torch.Tensor, lane, scale: float, window: int = 0,
                         n_splits: Optional[int] = None, tensor_cores: Optional[bool] = None,
                         out_compute_dtype: bool = False) -> torch.Tensor:
        """q_lat fp32 [tokens, heads, rank] over the lane's cached latents (one row per token, shared by all heads
        as key and as value) -> [tokens, heads, rank], the softmax-weighted sums of latents, fp32 (or, from the
        tensor-core kernel with ``out_compute_dtype``, bf16).  bf16 latents of a rank that is a multiple of 16 go to the
        tensor-core kernel (``tensor_cores`` False keeps the fp32 kernel)."""
        self._f32(q_lat, "latent queries")
        n, H, R = q_lat.shape
        mma_ok = self.latent_attention_on_tensor_cores(R)
        narrow = bool(out_compute_dtype) and mma_ok and tensor_cores is not False
        out = self.empty(n, H, R, dtype=self.dtype if narrow else torch.float32)
        if tensor_cores and not mma_ok:
            raise ValueError("the tensor-core latent attention takes bf16 latents of a rank that is a multiple of 16 up to 512")
        if mma_ok and tensor_cores is not False:
            if n_splits is None:
                n_splits = self.latent_attention_splits(ctx, n, H, int(window))
            scratch = None
            if n_splits > 1:
                scratch = self.empty(int(self.lib.cpm_latent_attention_scratch_floats(n, H, R, n_splits)), dtype=torch.float32)
            check(self.lib.cpm_latent_attention_mma(_ptr(q_lat), _ptr(lane.k), _ptr(out), 1 if narrow else 0, _ptr(scratch), _ptr(ctx.positions),
                                                    _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                                    lane.page_table.shape[1], int(window), n, H, R, float(scale), n_splits,
                                                    self._stream()), f"latent attention on tensor cores (rank {R}, {H} heads)")
            if n_splits > 1:
                LAUNCHES_EXTRA[0] += 1
            return out
        check(self.lib.cpm_latent_attention(_ptr(q_lat), _ptr(lane.k), _ptr(out), _ptr(ctx.positions), _ptr(ctx.token_seq),
                                            _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1], int(window),
                                            n, H, R, float(scale), self.code, self._stream()),
              f"latent attention (rank {R}, {H} heads)")
        return out

    # ---- matrix products ----
    SKINNY_MAX_ROWS = int(os.environ.get("CPMCU_SKINNY_MAX_ROWS", "8"))   # most rows the weight-streaming product takes
    # From this many rows on the gated product runs on the tcgen05 kernel.  Its 128-row tiles are mostly empty for a
    # decode batch, but the product is bound by streaming the weights, not by the tensor cores: at 16 to 128 rows
    # it takes 51 us on the 8B gate_up shape (5.2 TB/s) with the activation applied in the epilogue, where the library
    # product takes 51 us and the activation kernel 4 us more.
    SKINNY_WIDE_BYTES = int(os.environ.get("CPMCU_SKINNY_WIDE_MB", "128")) << 20   # see _skinny_ok
    TCGEN05_MIN_ROWS = int(os.environ.get("CPMCU_TCGEN05_MIN_ROWS", "9"))
    MAX_DECODE_SPLITS = int(os.environ.get("CPMCU_MAX_SPLITS", "16"))     # most shares a sequence's pages are cut into
    LISTED_TILE_MIN_TOKENS = int(os.environ.get("CPMCU_LISTED_TILE_MIN", "32"))   # from here on prompt tokens share their blocks in tiles of eight
    SELECT_SCRATCH_BYTES = 64 << 20     # most scratch the sliced block selection may take (raw scores of all pooled keys)

    def _skinny_ok(self, M: int, K: int, N: int = 0) -> bool:
        """The weight-streaming product takes it: up to SKINNY_MAX_ROWS rows always; 9 to 16 rows (two tiles of token
        columns) while what its blocks read of the activations (every block all of them) stays small: at 16 rows
        the QKV, O and down products of the 8B sizes (not gate_up and the head), where it took 3.8 % off the step
        against the library's kernels (which stand outside the chain of dependent launches).  With four and eight tiles (up to 64 rows) the kernel
        lost to the library at every size tried, the 0.5B sizes included, and is not built."""
        if self.code != BF16 or K % 32 != 0:
            return False
        if M <= self.SKINNY_MAX_ROWS:
            return True
        return 0 < N and M <= 16 and -(-N // 16) * M * K * 2 <= self.SKINNY_WIDE_BYTES

    def linear(self, a: torch.Tensor, w: torch.Tensor, alpha: float = 1.0,
               out_f32: bool = False, result: bool = False) -> torch.Tensor:
        """alpha * a[M,K] @ w[N,K]^T -> [M,N] in the compute dtype, or fp32 when out_f32.  ``result``: the
        product is handed to the step's caller (see ``result``)."""
        self._act(a, "linear input")
        self._act(w, "linear weight")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise ValueError(f"linear: input [*, {K}] against weight {tuple(w.shape)}")
        make = self.result if result else self.empty
        if self.code == F32:
            c = make(M, N, dtype=torch.float32)
            check(self.lib.cpm_gemm_f32(_ptr(a), _ptr(w), _ptr(c), M, N, K, K, K, N, float(alpha), self._stream()),
                  "fp32 matrix product")
            return c
        if self._skinny_ok(M, K, N):
            c = make(M, N, dtype=torch.float32 if out_f32 else self.dtype)
            check(self.lib.cpm_gemm_skinny_bf16(_ptr(w), _ptr(a), _ptr(c), M, N, K, float(alpha), 1 if out_f32 else 0,
                                                self._stream()), "skinny matrix product")
            return c
        c = make(M, N, dtype=torch.float32 if out_f32 else self.dtype)
        self._library_mm(a, w, c)
        if alpha != 1.0:
            c.mul_(alpha)
        return c

    def _library_mm(self, a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> None:
        """c = a @ w^T by the library (cuBLAS through torch), into a tensor of this library's own."""
        if c.dtype == a.dtype:
            torch.mm(a, w.t(), out=c)
        else:
            torch.mm(a, w.t(), out_dtype=c.dtype, out=c)

    def linear_tcgen05(self, a: torch.Tensor, w: torch.Tensor, gated: bool = False, pair: bool = False,
                       epilogue: int = 2) -> torch.Tensor:
        """a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA operands, TMEM accumulator); with ``gated`` the
        weight is a gate_up matrix interleaved in blocks of 8 and the result is act(gate) * up, [M, N/2] (``epilogue`` 2:
        SiLU, 3: the tanh form of GELU).
        ``pair``: two blocks work on one 256 x 256 tile (cta_group::2)."""
        self._act(a, "linear input")
        self._act(w, "linear weight")
        M, K = a.shape
        N = w.shape[0]
        out = self.empty(M, N // 2 if gated else N)
        entry = self.lib.cpm_gemm_bf16_tcgen05_pair if pair else self.lib.cpm_gemm_bf16_tcgen05
        check(entry(_ptr(a), _ptr(w), _ptr(out), M, N, K, int(epilogue) if gated else 0, self.sm_count, self._stream()),
              f"tcgen05 matrix product [{M}x{K}] x [{N}x{K}]^T")
        return out

    def tcgen05_error(self) -> int:
        """Error code the tcgen05 product kernel recorded since the last call (0 = none); synchronises."""
        return int(self.lib.cpm_gemm_tcgen05_error())

    def act_mul(self, gu: torch.Tensor, interleave: int, activation: int) -> torch.Tensor:
        """gu [tokens, 2*inter] -> act(gate) * up, [tokens, inter], for any activation code (0 SiLU, 1 tanh-GELU)."""
        self._act(gu, "gate_up")
        n, two_i = gu.shape
        h = self.empty(n, two_i // 2)
        check(self.lib.cpm_act_mul(_ptr(gu), _ptr(h), n, two_i // 2, interleave, int(activation), self.code, self._stream()),
              "act_mul")
        return h

    GATED_EPILOGUES = {0: 2, 1: 3}      # activation code -> the product kernels' gated epilogue (SiLU, tanh-GELU)

    def gated_linear(self, a: torch.Tensor, w_gate_up: torch.Tensor, interleave: int, activation: int = 0) -> torch.Tensor:
        """act(a @ gate^T) * (a @ up^T) for a gate_up matrix [2*inter, K] laid out as ``interleave`` says; the
        activation is SiLU (code 0) or the tanh form of GELU (code 1).  The weight-streaming product (few rows) and the
        tcgen05 product (many rows) apply it in their epilogues; otherwise a kernel of its own follows the product."""
        M, K = a.shape
        epilogue = self.GATED_EPILOGUES[int(activation)]
        if interleave == 8 and self._skinny_ok(M, K, w_gate_up.shape[0]) and w_gate_up.shape[0] % 16 == 0:
            self._act(a, "linear input")
            self._act(w_gate_up, "gate_up weight")
            h = self.empty(M, w_gate_up.shape[0] // 2)
            check(self.lib.cpm_gemm_skinny_bf16(_ptr(w_gate_up), _ptr(a), _ptr(h), M, w_gate_up.shape[0], K, 1.0, epilogue,
                                                self._stream()), "gated skinny matrix product")
            return h
        few_tiles = M < 256 and w_gate_up.shape[0] // 256 < self.sm_count // 2     # a decode batch on a narrow model: too few blocks
        if (self.code == BF16 and interleave == 8 and self.use_tcgen05 and M >= self.TCGEN05_MIN_ROWS and K % 64 == 0
                and w_gate_up.shape[0] % 32 == 0 and a.data_ptr() % 16 == 0 and not few_tiles):
            # many rows (prefill): the tcgen05 product applies the activation in its epilogue
            return self.linear_tcgen05(a, w_gate_up, gated=True, pair=self.tcgen05_pair, epilogue=epilogue)
        if activation == 0:
            return self.silu_mul(self.linear(a, w_gate_up), interleave)
        return self.act_mul(self.linear(a, w_gate_up), interleave, activation)

    # ---- attention ----
    def rope_store(self, qkv: torch.Tensor, n_heads: int, n_kv: int, d: int, positions: torch.Tensor,
                   token_seq: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                   k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   inv_freq: Optional[torch.Tensor], magnitude: float, rot_dim: int) -> torch.Tensor:
        """Rotates q and k of qkv [tokens, (heads+2*kv)*d], stores k and v into the cache pages of
        each token's sequence, and returns the rotated q [tokens, heads, d]."""
        self._act(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (n_heads + 2 * n_kv) * d:
            raise ValueError("qkv row size does not match the head counts")
        if inv_freq is not None:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != rot_dim // 2:
                raise ValueError("inv_freq needs rot_dim/2 entries")
        if k_cache is not None:
            self._act(k_cache, "key cache")
            self._act(v_cache, "value cache")
        q = self.empty(n, n_heads, d)
        check(self.lib.cpm_rope_store(_ptr(qkv), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(positions),
                                      _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                      _ptr(inv_freq), float(magnitude), n, n_heads, n_kv, d, rot_dim, self.code,
                                      self._stream()), "rope_store")
        return q

    def attention_generic(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          positions: torch.Tensor, token_seq: torch.Tensor, slots: torch.Tensor,
                          page_table: torch.Tensor, n_kv: int, scale: float, window: int = 0,
                          block_list: Optional[torch.Tensor] = None, block_size: int = 0) -> torch.Tensor:
        """q [tokens, heads, d] against the cached keys of each token's sequence -> [tokens, heads*d]."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        out = self.empty(n, n_heads * d)
        list_cap = 0
        if block_list is not None:
            self._i32(block_list, "block list")
            list_cap = block_list.shape[-1]
        check(self.lib.cpm_attention_generic(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                             _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                             _ptr(block_list), list_cap, block_size, window, n, n_heads, n_kv, d,
                                             float(scale), self.code, self._stream()),
              f"attention (head_dim {d}, {n_heads} heads, {n_kv} kv heads)")
        return out

    # ---- sampling ----
    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               top_p: Optional[torch.Tensor] = None, seed: int = 0, seq_key: Optional[torch.Tensor] = None,
               step_key: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits [rows, vocab] -> int32 [rows]; greedy where temperature is absent or 0."""
        self._f32(logits, "logits")
        rows, vocab = logits.shape
        if out is None:
            out = self.result(rows, dtype=torch.int32)
        check(self.lib.cpm_sample_rows(_ptr(logits), logits.stride(0), rows, vocab, _ptr(out), _ptr(temperature),
                                       _ptr(top_p), ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), _ptr(seq_key),
                                       _ptr(step_key), self._stream()), "sample")
        return out

    def attention(self, ctx, q: torch.Tensor, lane, n_kv: int, scale: float, window: int = 0,
                  block_list: Optional[torch.Tensor] = None, block_size: int = 0) -> torch.Tensor:
        """Attention of the step's queries over their sequences' cached keys; picks the kernel."""
        n, n_heads, d = q.shape
        if self.code == BF16 and block_list is None and not window and d in FAST_HEAD_DIMS:
            if ctx.is_decode:
                return self.decode_attention(q, lane.k, lane.v, ctx.kv_len_dev, ctx.slot_dev, lane.page_table,
                                             n_kv, scale)
            tiles = ctx.q_tiles
            if (tiles is not None and self.use_tcgen05_attention and (n_heads // n_kv) % 2 == 0
                    and (d == 128 or (d == 64 and ctx.max_kv_len >= 1024))):      # short prompts of head size 64: the smaller tiles win
                return self.prefill_attention_tcgen05(q, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev,
                                                      lane.page_table, n_kv, scale,
                                                      self.prefill_key_shares(ctx.q_lens, ctx.max_kv_len, n_heads))
            if tiles is not None:
                return self.prefill_attention(q, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev,
                                              lane.page_table, n_kv, scale)
        if (self.code == BF16 and block_list is not None and block_size == PAGE_TOKENS and not window
                and d in FAST_HEAD_DIMS):
            return self.listed_attention(q, lane.k, lane.v, ctx.positions, ctx.token_seq, ctx.slot_dev,
                                         lane.page_table, block_list, n_kv, scale,
                                         tiles=not ctx.is_decode and n >= self.LISTED_TILE_MIN_TOKENS)
        return self.attention_generic(q, lane.k, lane.v, ctx.positions, ctx.token_seq, ctx.slot_dev,
                                      lane.page_table, n_kv, scale, window, block_list, block_size)

    # ---- block-sparse selection ----
    def pool_keys(self, ctx, lane, n_kv: int, d: int, kernel: int, stride: int) -> None:
        """Stores the mean-pooled keys whose windows this step's tokens complete."""
        check(self.lib.cpm_pool_keys(_ptr(lane.k), _ptr(lane.pooled), _ptr(ctx.positions), _ptr(ctx.token_seq),
                                     _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1],
                                     ctx.n_tokens, n_kv, d, kernel, stride, self.code, self._stream()), "pool_keys")

    def select_blocks(self, ctx, q: torch.Tensor, lane, n_kv: int, scale: float, sparse) -> Tuple[torch.Tensor, int]:
        """(block list int32 [tokens, kv_heads, cap], block size) for the step's queries."""
        n, n_heads, d = q.shape
        bs, stride = sparse["block_size"], sparse["kernel_stride"]
        local_blocks = sparse["window_size"] // bs
        cap = sparse["topk"] + local_blocks + 2
        # an upper bound on the pooled keys a query sees; it sizes the sort of the candidate blocks (8 bytes of shared
        # memory per block), not the walk over the pooled keys, which follows each query's own position
        longest = ctx.max_kv_len          # in a recorded step an upper bound (the cache's capacity per sequence, or less)
        max_entries = max(1, longest // stride + 1)
        lists = self.empty(n, n_kv, cap, dtype=torch.int32)
        # few queries (a decode step): share every query's pooled keys out over many blocks, in two kernels
        scratch, n_slices = None, 0
        units = n * n_kv
        if (self.code == BF16 and units * 2 <= self.sm_count and n_heads // n_kv <= 16 and d in FAST_HEAD_DIMS
                and units * max_entries * 64 <= self.SELECT_SCRATCH_BYTES):
            n_slices = max(1, min(2 * self.sm_count // units, (max_entries + 63) // 64))
            scratch = self.empty(self.lib.cpm_select_blocks_scratch_floats(n, n_kv, max_entries, n_slices), dtype=torch.float32)
        check(self.lib.cpm_select_blocks(_ptr(q), _ptr(lane.pooled), _ptr(ctx.positions), _ptr(ctx.token_seq),
                                         _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1],
                                         _ptr(lists), cap, n, n_heads, n_kv, d, float(scale), sparse["kernel_size"],
                                         stride, bs, sparse.get("init_blocks", 1), sparse["topk"], local_blocks,
                                         sparse.get("dense_len", 0), max_entries, self.code, _ptr(scratch), n_slices,
                                         self._stream()),
              f"select_blocks ({max_entries} pooled keys)")
        if scratch is not None:
            LAUNCHES_EXTRA[0] += 1
        return lists, bs

    def advance_decode(self, ids, positions, kv_len, step_key, sampled, live) -> None:
        check(self.lib.cpm_advance_decode(_ptr(ids), _ptr(positions), _ptr(kv_len), _ptr(step_key), _ptr(sampled),
                                          _ptr(live), ids.numel(), self._stream()), "advance_decode")

    # ---- bf16 tensor-core attention ----
    def decode_splits(self, n_seqs: int, n_heads: int, n_kv: int) -> int:
        """How many shares a sequence's pages are cut into: the decode attention kernel holds one
        block per SM (its page buffers fill the shared memory), so aim at one wave of blocks."""
        m_tiles = (n_heads // n_kv + 15) // 16
        units = max(1, n_seqs * n_kv * m_tiles)
        return max(1, min(self.MAX_DECODE_SPLITS, self.sm_count // units))

    def decode_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len: torch.Tensor,
                         slots: torch.Tensor, page_table: torch.Tensor, n_kv: int, scale: float,
                         n_splits: Optional[int] = None, out: Optional[torch.Tensor] = None, v_shift: int = 0,
                         v_runs: int = 1) -> torch.Tensor:
        """One query token per sequence: q [seqs, heads, d] -> [seqs, heads*d].  ``v_shift``: the values come from
        key-value head (kv head + v_shift) mod n_kv instead of the keys' own.  ``v_runs`` > 1: one launch does the runs
        with shifts 0 .. v_runs - 1; the result is [v_runs, seqs, heads*d]."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        rows = n * max(1, int(v_runs))
        if n_splits is None:
            n_splits = self.decode_splits(rows, n_heads, n_kv)
        floats = self.lib.cpm_decode_attention_scratch_floats(rows, n_heads, n_kv, d, n_splits)
        scratch = self.empty(floats, dtype=torch.float32)
        if out is None:
            out = self.empty(rows, n_heads * d) if v_runs <= 1 else self.empty(v_runs, n, n_heads * d)
        if v_shift or v_runs > 1:
            check(self.lib.cpm_decode_attention_bf16_vshift(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(kv_len),
                                                            _ptr(slots), _ptr(page_table), page_table.shape[1], _ptr(scratch),
                                                            n, n_heads, n_kv, d, n_splits, float(scale), int(v_shift),
                                                            max(1, int(v_runs)), self._stream()),
                  f"decode attention (head_dim {d}, values shifted)")
        else:
            check(self.lib.cpm_decode_attention_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(kv_len),
                                                     _ptr(slots), _ptr(page_table), page_table.shape[1], _ptr(scratch),
                                                     n, n_heads, n_kv, d, n_splits, float(scale), self._stream()),
                  f"decode attention (head_dim {d})")
        if n_splits > 1:
            LAUNCHES_EXTRA[0] += 1       # the launcher starts two kernels: the shares, then their combination
        return out

    FUSED_ROPE_HEAD_DIMS = (64, 128)      # head sizes whose rotary pairs lie in one thread's fragments of the decode kernel

    def fused_decode_ok(self, ctx, d: int, rot_dim: int, window: int, sparse) -> bool:
        """Whether a decode step's rotation and cache store are done by the attention kernel itself.  It saves a
        launch, which counts where launches are what a step waits for (steps that are not recorded into a graph).
        Inside a graph the separate rotary kernel overlaps with its neighbours and the fused kernel is 0.7 % slower
        on the 8B decode step (3.537 against 3.501 ms at batch 8), so recorded steps keep the two kernels.
        CPMCU_FUSED_ROPE=1 / 0 forces the choice."""
        forced = os.environ.get("CPMCU_FUSED_ROPE")
        want = (forced != "0") if forced is not None else not ctx.captured
        return (want and self.code == BF16 and ctx.is_decode and not window and sparse is None
                and d in self.FUSED_ROPE_HEAD_DIMS and rot_dim in (0, d))

    def decode_attention_rope(self, qkv: torch.Tensor, lane, kv_len: torch.Tensor, slots: torch.Tensor, n_heads: int,
                              n_kv: int, d: int, scale: float, inv_freq: Optional[torch.Tensor], magnitude: float,
                              write_cache: bool, n_splits: Optional[int] = None) -> torch.Tensor:
        """A decode step's attention straight from the fused product qkv [seqs, (heads + 2 kv) * d]: the kernel
        rotates q and the new key (position = keys - 1), stores the new key and value into the sequence's page (when
        ``write_cache``) and attends.  One launch less than rope_store followed by decode_attention."""
        self._act(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (n_heads + 2 * n_kv) * d:
            raise ValueError("qkv row size does not match the head counts")
        if inv_freq is not None:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != d // 2:
                raise ValueError("inv_freq needs head_dim/2 entries")
        if n_splits is None:
            n_splits = self.decode_splits(n, n_heads, n_kv)
        floats = self.lib.cpm_decode_attention_scratch_floats(n, n_heads, n_kv, d, n_splits)
        scratch = self.empty(floats, dtype=torch.float32)
        out = self.empty(n, n_heads * d)
        check(self.lib.cpm_decode_attention_rope_bf16(_ptr(qkv), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(kv_len),
                                                      _ptr(slots), _ptr(lane.page_table), lane.page_table.shape[1],
                                                      _ptr(scratch), n, n_heads, n_kv, d, n_splits, float(scale),
                                                      _ptr(inv_freq), float(magnitude), 1 if write_cache else 0,
                                                      self._stream()), f"decode attention with rotation (head_dim {d})")
        if n_splits > 1:
            LAUNCHES_EXTRA[0] += 1
        return out

    def prefill_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles,
                          cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                          n_kv: int, scale: float, out: Optional[torch.Tensor] = None, v_shift: int = 0) -> torch.Tensor:
        """q [tokens, heads, d] packed by sequence -> [tokens, heads*d]; tiles = (tile_seq, tile_row, count)
        lists the query tiles of PREFILL_TILE_ROWS tokens.  ``v_shift``: as in ``decode_attention``."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        tile_seq, tile_row, n_tiles = tiles
        if out is None:
            out = self.empty(n, n_heads * d)
        check(self.lib.cpm_prefill_attention_bf16_vshift(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq),
                                                         _ptr(tile_row), n_tiles, _ptr(cu_q), _ptr(kv_len), _ptr(slots),
                                                         _ptr(page_table), page_table.shape[1], n_heads, n_kv, d,
                                                         float(scale), int(v_shift), self._stream()),
              f"prefill attention (head_dim {d})")
        return out


    def prefill_attention_tcgen05(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tiles,
                                  cu_q: torch.Tensor, kv_len: torch.Tensor, slots: torch.Tensor,
                                  page_table: torch.Tensor, n_kv: int, scale: float, n_splits: int = 1,
                                  out: Optional[torch.Tensor] = None, v_shift: int = 0) -> torch.Tensor:
        """The same as ``prefill_attention`` on the tcgen05 tensor cores: head size 128 or 64 and an even number
        of query heads per key/value head.  ``n_splits`` > 1 shares the keys of every tile out over that many
        blocks (a short chunk after a long history would otherwise keep few SMs busy for long)."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        tile_seq, tile_row, n_tiles = tiles
        if out is None:
            out = self.empty(n, n_heads * d)
        scratch = self.empty(n_splits * n * n_heads * (d + 2), dtype=torch.float32) if n_splits > 1 else None
        check(self.lib.cpm_prefill_attention_tcgen05_vshift(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq),
                                                            _ptr(tile_row), n_tiles, _ptr(cu_q), _ptr(kv_len), _ptr(slots),
                                                            _ptr(page_table), page_table.shape[1], n, k_cache.shape[0],
                                                            n_heads, n_kv, d, float(scale), _ptr(scratch), n_splits,
                                                            int(v_shift), self._stream()),
              f"tcgen05 prefill attention (head_dim {d})")
        return out

    def prefill_key_shares(self, q_lens, max_kv_len: int, n_heads: int) -> int:
        """How many blocks share the keys of a query tile in the tcgen05 attention: one, unless the step's 128-token
        tiles times head pairs leave most SMs idle and there are enough keys (at least 8 steps of 128 per share)."""
        blocks = sum((int(n) + 127) // 128 for n in q_lens) * max(1, n_heads // 2)
        steps = (int(max_kv_len) + 127) // 128
        if blocks * 2 > self.sm_count or steps < 16:
            return 1
        return max(1, min(self.sm_count // blocks, steps // 8, 16))

    def attention_tcgen05_error(self) -> int:
        """Error code the tcgen05 attention kernel recorded since the last call (0 = none); synchronises."""
        return int(self.lib.cpm_attention_tcgen05_error())

    def raise_on_kernel_error(self) -> None:
        """The tcgen05 kernels bound every wait and record a code instead of hanging; this turns a recorded
        code into an exception.  It synchronises the device: call it where the host waits anyway."""
        gemm, attn = self.tcgen05_error(), self.attention_tcgen05_error()
        if gemm or attn:
            raise RuntimeError(f"a tcgen05 kernel gave up waiting on a barrier (product: code {gemm}, attention: code "
                               f"{attn}); the results of this step are not valid")
        self.raise_on_bounds_error()
        arena = self.workspace.persistent.arena if self.workspace is not None else None
        if arena is not None and arena.guards:
            arena.check_guards()
        if int(self.lib.cpm_listed_tile_error()):
            raise RuntimeError("the block-list attention of a prompt chunk gave up waiting on a barrier; the results of "
                               "this step are not valid")
        if int(self.lib.cpm_select_blocks_error()):
            raise RuntimeError("block selection met a query with more candidate key blocks than the launch made room "
                               "for (a sequence longer than the bound the step gave); the results of this step are not valid")

    # ---- several residual streams ----
    def hyper_fan_out(self, x: torch.Tensor, n_streams: int) -> torch.Tensor:
        """fp32 [tokens, hidden] -> fp32 [tokens, streams, hidden], every stream a copy of x."""
        self._f32(x, "residual stream")
        n, hidden = x.shape
        X = self.empty(n, n_streams, hidden, dtype=torch.float32)
        check(self.lib.cpm_hyper_fan_out(_ptr(x), _ptr(X), n, n_streams, hidden, self._stream()), "hyper_fan_out")
        return X

    def hyper_step(self, X: torch.Tensor, write=None, read=None, eps: float = 0.0, total: Optional[torch.Tensor] = None
                   ) -> Optional[torch.Tensor]:
        """One pass over the residual streams X fp32 [tokens, streams, hidden], in place.  ``write`` = (y, mix, out):
        X_r <- sum_s mix[s][r] X_s + out[r] * y.  ``read`` = (in, gain): returns rms_norm(sum_s in[s] X_s) * gain in the
        compute dtype.  ``total`` (fp32 [tokens, hidden]) receives the sum of the streams."""
        self._f32(X, "residual streams")
        n, S, hidden = X.shape
        y = mix = out_w = in_w = gain = h = None
        if write is not None:
            y, mix, out_w = write
            self._act(y, "sublayer output")
            if y.shape != (n, hidden):
                raise ValueError(f"sublayer output {tuple(y.shape)} does not match the streams {tuple(X.shape)}")
            self._f32(mix, "stream mix")
            self._f32(out_w, "stream output weights")
        if read is not None:
            in_w, gain = read
            self._f32(in_w, "stream input weights")
            self._f32(gain, "norm gain")
            h = self.empty(n, hidden)
        if total is not None:
            self._f32(total, "sum of the streams")
        check(self.lib.cpm_hyper_step(_ptr(X), _ptr(y), _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(gain), float(eps), _ptr(h),
                                      _ptr(total), n, S, hidden, self.code, self._stream()), f"hyper_step ({S} streams)")
        return h

    # ---- linear recurrences with a matrix state ----
    def linear_recurrence(self, ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor,
                          beta: Optional[torch.Tensor], state: torch.Tensor, heads: int, qk_heads: int, d: int, dv: int,
                          q_scale: float, vector_decay: bool = False) -> torch.Tensor:
        """S <- diag(decay) S; u = v (or beta (v - S^T k) when ``beta`` is given); S <- S + k u^T; o = S^T q * q_scale, per
        head and token, in 32-bit.  q, k: fp32 views [tokens, qk_heads * d]; v: [tokens, heads * dv]; decay: [tokens, heads], or
        with ``vector_decay`` [tokens, heads * d] (one number per key channel); beta: [tokens, heads]; rows may be slices of wider rows (unit
        stride inside a row).  state fp32 [slots, heads, d, dv], read at a sequence's first token of the step (zeros at
        position 0) and written at its last.  Returns fp32 [tokens, heads, dv]."""
        n = q.shape[0]
        for t, what, width in ((q, "q", qk_heads * d), (k, "k", qk_heads * d), (v, "v", heads * dv)):
            if t.dtype != torch.float32 or t.shape != (n, width) or t.stride(1) != 1:
                raise ValueError(f"linear_recurrence: {what} must be fp32 [tokens, {width}] with unit stride inside a row")
        if q.stride(0) != k.stride(0):
            raise ValueError("linear_recurrence: q and k must have the same row stride")
        vector = bool(vector_decay)
        if decay.shape != (n, heads * d if vector else heads) or decay.dtype != torch.float32 or decay.stride(1) != 1:
            raise ValueError("linear_recurrence: decay must be fp32 [tokens, heads] or, with vector_decay, [tokens, heads * d]")
        if beta is not None and (beta.dtype != torch.float32 or beta.shape != (n, heads) or beta.stride(1) != 1):
            raise ValueError("linear_recurrence: beta must be fp32 [tokens, heads]")
        self._f32(state, "recurrence state")
        if tuple(state.shape[1:]) != (heads, d, dv):
            raise ValueError(f"linear_recurrence: state {tuple(state.shape)} is not [slots, {heads}, {d}, {dv}]")
        out = self.empty(n, heads, dv, dtype=torch.float32)
        check(self.lib.cpm_linear_recurrence(_ptr(q), _ptr(k), q.stride(0), _ptr(v), v.stride(0), _ptr(decay), decay.stride(0),
                                             1 if vector else 0, _ptr(beta), beta.stride(0) if beta is not None else 0,
                                             _ptr(state), _ptr(ctx.positions), _ptr(ctx.cu_q), _ptr(ctx.slot_dev), _ptr(out),
                                             ctx.n_seqs, heads, qk_heads, d, dv, float(q_scale), self._stream()),
              f"linear_recurrence ({heads} heads, {d} x {dv})")
        return out

    def conv_prepare(self, ctx, proj: torch.Tensor, taps: torch.Tensor, conv_state: torch.Tensor, a_log: torch.Tensor,
                     dt_bias: torch.Tensor, b_col: int, a_col: int, heads: int, qk_heads: int, d: int, dv: int, unit_eps: float,
                     head_decay: bool = True):
        """proj fp32 [tokens, N] whose rows begin [q | k | v] and hold the raw gates at columns ``b_col`` and ``a_col``
        (one per head): short causal convolution (taps fp32 [channels, K], the last column the current token's) and SiLU
        on q, k, v; q and k heads scaled to unit length; beta = sigmoid(b), decay = exp(-exp(a_log) softplus(a + dt_bias)).
        conv_state fp32 [slots, K-1, channels] gives the inputs before the step and takes those after it.  Returns fp32
        (q [tokens, qk_heads*d], k, v [tokens, heads*dv], beta [tokens, heads], decay [tokens, heads]); without
        ``head_decay`` no decay is formed (None; ``a_log``, ``dt_bias`` and ``a_col`` are not read)."""
        self._f32(proj, "projections")
        self._f32(taps, "convolution taps")
        self._f32(conv_state, "convolution state")
        n = proj.shape[0]
        C, K = taps.shape
        if C != 2 * qk_heads * d + heads * dv or tuple(conv_state.shape[1:]) != (max(K - 1, 1), C):
            raise ValueError("conv_prepare: taps [channels, K] and state [slots, K-1, channels] do not match the head sizes")
        qo = self.empty(n, qk_heads * d, dtype=torch.float32)
        ko = self.empty(n, qk_heads * d, dtype=torch.float32)
        vo = self.empty(n, heads * dv, dtype=torch.float32)
        beta = self.empty(n, heads, dtype=torch.float32)
        decay = self.empty(n, heads, dtype=torch.float32) if head_decay else None
        check(self.lib.cpm_conv_prepare(_ptr(proj), proj.stride(0), _ptr(taps), _ptr(conv_state), _ptr(ctx.positions),
                                        _ptr(ctx.token_seq), _ptr(ctx.cu_q), _ptr(ctx.slot_dev), _ptr(qo), _ptr(ko), _ptr(vo),
                                        _ptr(beta), _ptr(decay), _ptr(a_log), _ptr(dt_bias), int(b_col), int(a_col), n, ctx.n_seqs,
                                        heads, qk_heads, d, dv, K, float(unit_eps), self._stream()), "conv_prepare")
        if K > 1:
            LAUNCHES_EXTRA[0] += 1
        return qo, ko, vo, beta, decay

    def channel_decay(self, z: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, heads: int, d: int) -> torch.Tensor:
        """In place on fp32 [tokens, heads * d]: exp(-exp(a_log[h]) * softplus(z + dt_bias)), a decay per head and key
        channel (a_log fp32 [heads], dt_bias fp32 [heads * d])."""
        self._f32(z, "decay logits")
        self._f32(a_log, "A_log")
        self._f32(dt_bias, "dt_bias")
        if z.shape[1] != heads * d or a_log.numel() != heads or dt_bias.numel() != heads * d:
            raise ValueError("channel_decay: logits [tokens, heads * d], a_log [heads], dt_bias [heads * d]")
        check(self.lib.cpm_channel_decay(_ptr(z), _ptr(a_log), _ptr(dt_bias), z.shape[0], heads, d, self._stream()), "channel_decay")
        return z

    def sigmoid_power(self, z: torch.Tensor, bias: torch.Tensor, tau: float) -> torch.Tensor:
        """In place on fp32 [tokens, width]: sigmoid(z + bias)^(1/tau)."""
        self._f32(z, "decay logits")
        self._f32(bias, "decay bias")
        check(self.lib.cpm_sigmoid_power(_ptr(z), _ptr(bias), float(tau), z.shape[0], z.shape[1], self._stream()), "sigmoid_power")
        return z

    def gated_head_norm(self, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float,
                        gate_activation: str = "silu") -> torch.Tensor:
        """o fp32 [tokens, heads, dv], gate fp32 [tokens, heads*dv] (may be a slice of wider rows), weight fp32 [dv] ->
        rms_norm(o) * weight * act(gate) per head (act: "silu" or "sigmoid"), [tokens, heads*dv] in the compute dtype."""
        self._f32(o, "recurrence output")
        self._f32(weight, "head norm weight")
        n, heads, dv = o.shape
        if gate.dtype != torch.float32 or gate.shape != (n, heads * dv) or gate.stride(1) != 1:
            raise ValueError("gated_head_norm: the gate must be fp32 [tokens, heads*dv]")
        out = self.empty(n, heads * dv)
        check(self.lib.cpm_gated_head_norm(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), n, heads, dv, float(eps),
                                           {"silu": 0, "sigmoid": 1}[gate_activation], self.code, self._stream()), "gated_head_norm")
        return out

    GATE_ACTIVATIONS = {"silu": 0, "sigmoid": 1}

    def gated_group_norm(self, o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, group: int,
                         gate_activation: str = "silu") -> torch.Tensor:
        """As ``gated_head_norm`` with ``group`` heads normed together (``group`` = heads: all heads of a token as one
        vector), weight fp32 [group * dv], and the gate passed through SiLU or the sigmoid."""
        self._f32(o, "recurrence output")
        self._f32(weight, "group norm weight")
        n, heads, dv = o.shape
        if gate.dtype != torch.float32 or gate.shape != (n, heads * dv) or gate.stride(1) != 1:
            raise ValueError("gated_group_norm: the gate must be fp32 [tokens, heads*dv]")
        if heads % group or weight.numel() != group * dv:
            raise ValueError(f"gated_group_norm: {heads} heads in groups of {group} need a weight of {group * dv} numbers")
        out = self.empty(n, heads * dv)
        check(self.lib.cpm_gated_group_norm(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), n, heads, dv, int(group),
                                            self.GATE_ACTIVATIONS[gate_activation], float(eps), self.code, self._stream()),
              "gated_group_norm")
        return out

    def silu_columns(self, x: torch.Tensor, cols: int) -> torch.Tensor:
        """In place on fp32 rows: the first ``cols`` entries of every row pass through SiLU."""
        if x.dtype != torch.float32 or x.dim() != 2 or x.stride(1) != 1 or cols > x.shape[1]:
            raise ValueError("silu_columns: needs fp32 rows with unit stride inside a row")
        check(self.lib.cpm_silu_columns(_ptr(x), x.stride(0), x.shape[0], int(cols), self._stream()), "silu_columns")
        return x

    # ---- attention with capped scores, a window and a sink ----
    def qk_prepare_store(self, ctx, proj: torch.Tensor, lane, n_heads: int, n_kv: int, d: int, dv: int,
                         biases, inv_freq: Optional[torch.Tensor], rot_dim: int, unit_rms: bool, eps: float,
                         has_kv: bool = True, adjacent: bool = False, extra_cols: int = 0) -> torch.Tensor:
        """proj fp32 [tokens, heads*d + kv*d + kv*dv] (or [tokens, heads*d] without ``has_kv``): adds the biases
        (``biases`` = (q, k, v), fp32 or None each), rotates the first ``rot_dim`` channels of every q and k head
        (pairs (i, i + rot_dim/2), or (2i, 2i + 1) with ``adjacent``; angle position * inv_freq[i]), divides q and k heads by their root mean square
        (``unit_rms``), stores k and v into the lane's pages and returns q [tokens, heads, d] in the compute dtype."""
        self._f32(proj, "projections")
        n = proj.shape[0]
        if proj.shape[1] != n_heads * d + (n_kv * (d + dv) if has_kv else 0) + int(extra_cols):      # extra_cols: what the caller keeps behind them
            raise ValueError("qk_prepare_store: the projections' row size does not match the head counts")
        if inv_freq is not None:
            self._f32(inv_freq, "inv_freq")
            if inv_freq.numel() != rot_dim // 2:
                raise ValueError("inv_freq needs rot_dim/2 entries")
        bq, bk, bv = biases
        for b, what in ((bq, "q bias"), (bk, "k bias"), (bv, "v bias")):
            if b is not None:
                self._f32(b, what)
        q = self.empty(n, n_heads, d)
        check(self.lib.cpm_qk_prepare_store(_ptr(proj), proj.stride(0), _ptr(bq), _ptr(bk), _ptr(bv), _ptr(q),
                                            _ptr(lane.k) if has_kv else None, _ptr(lane.v) if has_kv else None,
                                            _ptr(ctx.positions), _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                            lane.page_table.shape[1], _ptr(inv_freq) if rot_dim else None, int(rot_dim),
                                            1 if adjacent else 0, 1 if unit_rms else 0, float(eps), n, n_heads, n_kv, d, dv,
                                            1 if has_kv else 0,
                                            self.code, self._stream()), "qk_prepare_store")
        return q

    def sink_attention(self, ctx, q: torch.Tensor, lane, n_kv: int, dv: int, scale: float, window: int = 0, cap: float = 0.0,
                       sink: bool = True, keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                       gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q [tokens, heads, d] over the lane's cached keys and values -> [tokens, heads*dv]: scores times ``scale``, capped
        by cap * tanh(s / cap) when ``cap`` > 0, keys 0 <= i - j < ``window`` (0: all before and at i) and, with a window,
        the keys j < ``keep_first`` too; softmax with exp(b_h) added to the denominator when ``sink`` (``sinks``: fp32
        [heads], the b_h; None: 0); head h's output times sigmoid(gate[t][h]) (``gate``: fp32 [tokens, heads], may be a
        slice of wider rows; None: none).  Picks the kernel: bf16 with head sizes the tensor-core kernels are built
        for goes to them (prompt tokens by the step's query tiles, anything else token by token); other sizes and the
        32-bit path go to the kernel of every size."""
        n, n_heads, d = q.shape
        if (self.code == BF16 and self.lib.cpm_sink_attention_bf16_sizes(d, dv)
                and os.environ.get("CPMCU_SINK_GENERIC", "0") != "1"):
            if (not ctx.is_decode and ctx.q_tiles is not None and ctx.max_q_len >= self.SINK_TCGEN05_MIN_ROWS
                    and self.use_tcgen05_attention and self.use_tcgen05_sink and d == dv and (n_heads // n_kv) % 2 == 0
                    and (d == 128 or (d == 64 and ctx.max_kv_len >= 1024))):
                return self.sink_attention_tcgen05(ctx, q, lane, n_kv, scale, window, cap, sink, keep_first, sinks, gate)
            return self.sink_attention_bf16(ctx, q, lane, n_kv, dv, scale, window, cap, sink, keep_first, sinks, gate)
        return self.sink_attention_generic(ctx, q, lane, n_kv, dv, scale, window, cap, sink, keep_first, sinks, gate)

    def _sink_extras(self, n: int, n_heads: int, window: int, keep_first: int, sinks, gate):
        """Checked (keep_first, sinks pointer, gate pointer, gate stride) of the sink attention kernels."""
        if sinks is not None:
            self._f32(sinks, "sink scores")
            if sinks.numel() != n_heads:
                raise ValueError("sink scores: one number per head")
        if gate is not None and (gate.dtype != torch.float32 or gate.shape != (n, n_heads) or gate.stride(1) != 1):
            raise ValueError("the output gate must be fp32 [tokens, heads]")
        return (int(keep_first) if window else 0, _ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0)

    SINK_TCGEN05_MIN_ROWS = 32   # prompt portions from this many tokens on take the tcgen05 kernel's 128-row tiles

    def sink_attention_tcgen05(self, ctx, q: torch.Tensor, lane, n_kv: int, scale: float, window: int, cap: float,
                               sink: bool, keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                               gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Prompt tokens on the tcgen05 kernel of ``prefill_attention_tcgen05`` (equal key and value head sizes of 128 or
        64, an even number of query heads per key-value head): the window moves a tile's first key step and masks its
        edge, the cap and the sink join the softmax threads' work.  The weights enter the second product as bf16."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        tile_seq, tile_row, n_tiles = ctx.q_tiles
        keep, p_sinks, p_gate, gate_stride = self._sink_extras(n, n_heads, window, keep_first, sinks, gate)
        out = self.empty(n, n_heads * d)
        keys = min(ctx.max_kv_len, int(window) + 128 + keep) if window else ctx.max_kv_len
        n_splits = self.prefill_key_shares(ctx.q_lens, keys, n_heads)
        scratch = self.empty(n_splits * n * n_heads * (d + 2), dtype=torch.float32) if n_splits > 1 else None
        check(self.lib.cpm_sink_attention_tcgen05(_ptr(q), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(tile_seq), _ptr(tile_row),
                                                  int(n_tiles), _ptr(ctx.cu_q), _ptr(ctx.kv_len_dev), _ptr(ctx.slot_dev),
                                                  _ptr(lane.page_table), lane.page_table.shape[1], n, lane.k.shape[0], n_heads,
                                                  n_kv, d, float(scale), int(window), float(cap), 1 if sink else 0, keep, p_sinks,
                                                  p_gate, gate_stride, _ptr(scratch), n_splits, self._stream()),
              f"tcgen05 sink attention (head_dim {d})")
        return out

    SINK_MAX_SPLITS = 16

    def sink_attention_splits(self, ctx, n_tokens: int, n_heads: int, n_kv: int, window: int) -> int:
        """Blocks that share the keys of a token taken alone: none while the tokens fill the device; else enough for
        about two blocks an SM, as long as each of a block's four warps keeps at least two steps of 32 keys."""
        blocks = n_tokens * n_kv * ((n_heads // n_kv + 15) // 16)
        if blocks * 2 > self.sm_count:
            return 1
        keys = min(window, ctx.max_kv_len) if window else ctx.max_kv_len      # in a recorded step an upper bound
        return max(1, min(self.SINK_MAX_SPLITS, 2 * self.sm_count // blocks, ((keys + 31) // 32) // 8))

    SINK_TILE_MIN_ROWS = 8       # shorter portions than this go token by token (a tile of 16 rows would be mostly empty)

    def sink_attention_bf16(self, ctx, q: torch.Tensor, lane, n_kv: int, dv: int, scale: float, window: int, cap: float,
                            sink: bool, keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                            gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The tensor-core kernels (bf16 operands; scores, cap, maxima, sums and accumulators fp32; a weight enters the
        product with the values as the sum of two bf16 numbers).  A warp owns 16 rows: query tokens of one head in a prompt
        (``ctx.q_tiles``), the query heads of one key-value head for a token taken alone."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        keep, p_sinks, p_gate, gate_stride = self._sink_extras(n, n_heads, window, keep_first, sinks, gate)
        out = self.empty(n, n_heads * dv)
        tiles = None if ctx.is_decode or ctx.max_q_len < self.SINK_TILE_MIN_ROWS else ctx.q_tiles
        tile_seq, tile_row, n_tiles = tiles if tiles is not None else (None, None, 0)
        n_splits, shares = 1, None
        if n_tiles == 0:
            n_splits = self.sink_attention_splits(ctx, n, n_heads, n_kv, int(window))
            if n_splits > 1:
                shares = self.empty(n_splits * n * n_heads * (dv + 2), dtype=torch.float32)
        check(self.lib.cpm_sink_attention_bf16(_ptr(q), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(tile_seq), _ptr(tile_row),
                                               int(n_tiles), _ptr(ctx.cu_q), _ptr(ctx.kv_len_dev), _ptr(ctx.positions),
                                               _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                               lane.page_table.shape[1], int(window), keep, n, n_heads, n_kv, d, dv, float(scale),
                                               float(cap), 1 if sink else 0, p_sinks, p_gate, gate_stride, _ptr(shares),
                                               n_splits, self._stream()),
              f"sink attention on tensor cores ({n_heads} heads, {d} / {dv})")
        return out

    def sink_attention_generic(self, ctx, q: torch.Tensor, lane, n_kv: int, dv: int, scale: float, window: int, cap: float,
                               sink: bool, keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                               gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The kernel of every size and both precisions (one warp per token and head, fp32 arithmetic)."""
        self._act(q, "q")
        n, n_heads, d = q.shape
        keep, p_sinks, p_gate, gate_stride = self._sink_extras(n, n_heads, window, keep_first, sinks, gate)
        out = self.empty(n, n_heads * dv)
        check(self.lib.cpm_sink_attention_generic(_ptr(q), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(ctx.positions),
                                                  _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                                  lane.page_table.shape[1], int(window), keep, n, n_heads, n_kv, d, dv,
                                                  float(scale), float(cap), 1 if sink else 0, p_sinks, p_gate, gate_stride,
                                                  self.code, self._stream()),
              f"sink attention ({n_heads} heads, {d} / {dv})")
        return out

    def dual_rmsnorm_mean(self, a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float) -> torch.Tensor:
        """(rms_norm(a) * wa + rms_norm(b) * wb) / 2 over the last axis, [tokens, hidden] in the compute dtype."""
        self._act(a, "left output")
        self._act(b, "right output")
        self._f32(wa, "left norm weight")
        self._f32(wb, "right norm weight")
        if a.shape != b.shape:
            raise ValueError("dual_rmsnorm_mean: the two outputs differ in shape")
        out = self.empty(*a.shape)
        check(self.lib.cpm_dual_rmsnorm_mean(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(out), a.shape[0], a.shape[1], float(eps),
                                             self.code, self._stream()), "dual_rmsnorm_mean")
        return out

    # ---- attention with weights mixed across heads ----
    def rope_store_dv(self, ctx, qkv: torch.Tensor, lane, n_heads: int, n_kv: int, d: int, dv: int,
                      inv_freq: Optional[torch.Tensor], rot_dim: int, write_cache: bool = True) -> torch.Tensor:
        """qkv [tokens, heads*d + kv*d + kv*dv]: rotates q and k (the first ``rot_dim`` dimensions of a head, pairs
        (i, i + rot_dim/2)), stores k and v into the lane's pages, returns the rotated q [tokens, heads, d]."""
        self._act(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (n_heads + n_kv) * d + n_kv * dv:
            raise ValueError("qkv row size does not match the head counts")
        q = self.empty(n, n_heads, d)
        check(self.lib.cpm_rope_store_dv(_ptr(qkv), _ptr(q), _ptr(lane.k) if write_cache else None,
                                         _ptr(lane.v) if write_cache else None, _ptr(ctx.positions), _ptr(ctx.token_seq),
                                         _ptr(ctx.slot_dev), _ptr(lane.page_table), lane.page_table.shape[1], _ptr(inv_freq), 1.0,
                                         n, n_heads, n_kv, d, dv, int(rot_dim), self.code, self._stream()), "rope_store_dv")
        return q

    TALKING_MAX_RUNS = 8      # most key-value heads for which the mix is built from runs of the plain attention kernels

    def talking_attention_on_tensor_cores(self, ctx, n_heads: int, n_kv: int, d: int, dv: int) -> bool:
        """bf16, equal key and value sizes that the tensor-core attention kernels are built for, few key-value heads, and
        a step they take (one token per sequence, or prompt tokens with query tiles)."""
        return (self.code == BF16 and d == dv and d in FAST_HEAD_DIMS and n_kv <= self.TALKING_MAX_RUNS
                and (ctx.is_decode or ctx.q_tiles is not None) and os.environ.get("CPMCU_TALKING_GENERIC", "0") != "1")

    def talking_attention(self, ctx, q: torch.Tensor, lane, n_kv: int, dv: int, scale: float, temp: torch.Tensor,
                          talk: torch.Tensor) -> torch.Tensor:
        """Causal softmax attention over the lane's cache with scores times ``scale * temp[head]`` and the softmax
        weights mixed across heads by ``talk`` [heads, heads] (row: the head that receives); q [tokens, heads, d] ->
        [tokens, heads*dv].  Picks the kernels: the mix is linear in the weights, o_h = sum_g talk[h][g] A[g][kv(h)] with
        A[g][c] head g's weights applied to the values of key-value head c, so n_kv runs of the plain tensor-core
        attention (run s reading the values s heads after the keys') and one mixing kernel give it; sizes and steps
        those kernels do not take, and the 32-bit path, go to the kernel that forms the mixed weights itself."""
        n, n_heads, d = q.shape
        if not self.talking_attention_on_tensor_cores(ctx, n_heads, n_kv, d, dv):
            return self.talking_attention_generic(ctx, q, lane, n_kv, dv, scale, temp, talk)
        self._act(q, "q")
        self._f32(temp, "head temperatures")
        self._f32(talk, "head mix")
        qs = self.empty(n, n_heads, d)
        check(self.lib.cpm_scale_heads_bf16(_ptr(q), _ptr(temp), _ptr(qs), n, n_heads, d, self._stream()), "scale_heads")
        parts = self.empty(n_kv, n, n_heads * d)
        tiles = ctx.q_tiles
        on_tcgen05 = (not ctx.is_decode and self.use_tcgen05_attention and (n_heads // n_kv) % 2 == 0
                      and (d == 128 or (d == 64 and ctx.max_kv_len >= 1024)))
        shares = self.prefill_key_shares(ctx.q_lens, ctx.max_kv_len, n_heads) if on_tcgen05 else 1
        if ctx.is_decode:          # all runs in one launch (and one combination of the keys' shares)
            self.decode_attention(qs, lane.k, lane.v, ctx.kv_len_dev, ctx.slot_dev, lane.page_table, n_kv, scale, out=parts,
                                  v_runs=n_kv)
        for s in range(n_kv if not ctx.is_decode else 0):
            if on_tcgen05:
                self.prefill_attention_tcgen05(qs, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev, lane.page_table,
                                               n_kv, scale, shares, out=parts[s], v_shift=s)
            else:
                self.prefill_attention(qs, lane.k, lane.v, tiles, ctx.cu_q, ctx.kv_len_dev, ctx.slot_dev, lane.page_table, n_kv,
                                       scale, out=parts[s], v_shift=s)
        out = self.empty(n, n_heads * d)
        check(self.lib.cpm_talk_mix_bf16(_ptr(parts), _ptr(talk), _ptr(out), n, n_heads, n_kv, d, self._stream()), "talk_mix")
        return out

    def talking_attention_generic(self, ctx, q: torch.Tensor, lane, n_kv: int, dv: int, scale: float, temp: torch.Tensor,
                                  talk: torch.Tensor) -> torch.Tensor:
        """The kernel that forms the mixed weights itself (two walks over a query's keys), any sizes, both precisions."""
        self._act(q, "q")
        self._f32(temp, "head temperatures")
        self._f32(talk, "head mix")
        n, n_heads, d = q.shape
        out = self.empty(n, n_heads * dv)
        check(self.lib.cpm_talking_attention(_ptr(q), _ptr(lane.k), _ptr(lane.v), _ptr(out), _ptr(ctx.positions),
                                             _ptr(ctx.token_seq), _ptr(ctx.slot_dev), _ptr(lane.page_table),
                                             lane.page_table.shape[1], _ptr(temp), _ptr(talk), n, n_heads, n_kv, d, dv,
                                             float(scale), self.code, self._stream()),
              f"talking-heads attention ({n_heads} heads, {d} / {dv})")
        return out

    # ---- routed experts ----
    def moe_route(self, logits: torch.Tensor, correction: Optional[torch.Tensor], n_experts: int, top: int, n_groups: int, keep: int,
                  gate_col: int = -1, bias: Optional[torch.Tensor] = None, top_first: bool = False, sigmoid: bool = False):
        """logits fp32 [tokens, >= experts] -> (chosen int32 [tokens, top], weights fp32 [tokens, top], sigmoid of column
        ``gate_col`` fp32 [tokens] or None).  Default rule: softmax over all experts, choice by score + ``correction``
        within the kept groups, weights the plain scores.  ``top_first``: choice by logit + ``bias`` (fp32 [experts] or
        None), weights the softmax over the chosen logits only.  ``sigmoid``: scores are the sigmoids of the logits, the
        largest are chosen and are the weights as they are."""
        self._f32(logits, "router logits")
        if top_first or sigmoid:
            if bias is not None:
                self._f32(bias, "router bias")
            if n_groups != 1:
                raise ValueError("moe_route: the rule that chooses first has no groups of experts")
        else:
            self._f32(correction, "router correction")
        n = logits.shape[0]
        chosen = self.empty(n, top, dtype=torch.int32)
        weights = self.empty(n, top, dtype=torch.float32)
        gate = self.empty(n, dtype=torch.float32) if gate_col >= 0 else None
        check(self.lib.cpm_moe_route(_ptr(logits), logits.shape[1], _ptr(correction), _ptr(chosen), _ptr(weights), _ptr(gate),
                                     int(gate_col), n, n_experts, top, n_groups, keep, _ptr(bias), 2 if sigmoid else (1 if top_first else 0),
                                     self._stream()),
              f"moe_route ({n_experts} experts, top {top})")
        return chosen, weights, gate

    MOE_PAIRWISE_MAX_PAIRS = int(os.environ.get("CPMCU_MOE_PAIRWISE_MAX", "96"))     # up to here a pair streams its expert alone

    def moe_experts(self, x: torch.Tensor, chosen: torch.Tensor, w_gate: Optional[torch.Tensor], w_up: torch.Tensor,
                    w_down: torch.Tensor, input_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [tokens, hidden]; chosen int32 [tokens, top]; stacks w_gate, w_up [experts, ff, hidden], w_down [experts,
        hidden, ff] -> every pair's expert output, [tokens * top, hidden] in the compute dtype.  An expert is
        down(silu(gate x) * up x), or without a gate stack (``w_gate`` None) down(relu(up (s x))^2) with s =
        ``input_scale`` [tokens, top] (fp32; None: 1), applied to the up product's result, which is linear in x."""
        self._act(x, "expert input")
        for w, what in ((w_gate, "gate stack"), (w_up, "up stack"), (w_down, "down stack")):
            if w is not None:
                self._act(w, what)
        n, hidden = x.shape
        top = chosen.shape[1]
        E, ff, _ = w_up.shape
        mode = 1 if w_gate is not None else 2
        first, second = (w_gate, w_up) if mode == 1 else (w_up, None)
        if input_scale is not None:
            self._f32(input_scale, "expert input scale")
            if mode == 1 or input_scale.shape != (n, top):
                raise ValueError("moe_experts: an input scale [tokens, top] goes with experts that have no gate stack")
        pairs = n * top
        h = self.empty(pairs, ff)
        y = self.empty(pairs, hidden)
        if (self.code == BF16 and pairs <= self.MOE_PAIRWISE_MAX_PAIRS and hidden % 8 == 0 and ff % 8 == 0
                and hidden <= 12288 and ff <= 12288):
            # few pairs (a decode step): every pair streams its expert's weights, no grouping
            check(self.lib.cpm_moe_pair_product(_ptr(x), _ptr(first), _ptr(second), _ptr(h), _ptr(chosen), pairs, top, ff, hidden, mode,
                                                _ptr(input_scale), self._stream()), "moe gate/up product by pair")
            check(self.lib.cpm_moe_pair_product(_ptr(h), _ptr(w_down), None, _ptr(y), _ptr(chosen), pairs, top, hidden, ff, 0,
                                                None, self._stream()), "moe down product by pair")
            return y
        offsets = self.empty(E + 1, dtype=torch.int32)
        order = self.empty(pairs, dtype=torch.int32)
        check(self.lib.cpm_moe_group(_ptr(chosen), pairs, E, _ptr(offsets), _ptr(order), self._stream()), "moe_group")
        check(self.lib.cpm_moe_expert_product(_ptr(x), _ptr(first), _ptr(second), _ptr(h), _ptr(offsets), _ptr(order), pairs, E, top,
                                              ff, hidden, mode, _ptr(input_scale), self.code, self._stream()), "moe gate/up product")
        check(self.lib.cpm_moe_expert_product(_ptr(h), _ptr(w_down), None, _ptr(y), _ptr(offsets), _ptr(order), pairs, E, top,
                                              hidden, ff, 0, None, self.code, self._stream()), "moe down product")
        return y

    def moe_combine(self, y: torch.Tensor, weights: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                    gate: Optional[torch.Tensor], top: Optional[int] = None) -> torch.Tensor:
        """out[t] = sum_k weights[t][k] * y[t*top + k] (+ gate[t] * shared[t]); without weights (``top`` given) the plain sum."""
        n, top = weights.shape if weights is not None else (y.shape[0] // int(top), int(top))
        hidden = y.shape[1]
        out = self.empty(n, hidden)
        check(self.lib.cpm_moe_combine(_ptr(y), _ptr(weights), _ptr(shared), _ptr(gate), _ptr(out), n, top, hidden, self.code,
                                       self._stream()), "moe_combine")
        return out

    # ---- the checked build (CPMCU_CHECK_BOUNDS=1) ----
    def set_page_limit(self, n_pages: int) -> None:
        """Tells the checked kernels how many pages the cache in use holds (no-op in the ordinary build)."""
        if (getattr(self.lib, "checked_files", None) and n_pages != getattr(self, "_page_limit", None)
                and not torch.cuda.is_current_stream_capturing()):
            for _, _, limit in self.lib.checked_files:
                limit(int(n_pages))
            self._page_limit = n_pages

    def raise_on_bounds_error(self) -> None:
        """The checked build's records: a page index or page number out of range that a kernel met (and did not
        follow).  Synchronises."""
        for name, error, _ in getattr(self.lib, "checked_files", None) or ():
            rec = (ctypes.c_int * 4)()
            if error(ctypes.byref(rec)):
                what = "a page-table index beyond the table" if rec[0] == 1 else "a page number beyond the cache"
                raise RuntimeError(f"checked build: a kernel of {name}.cu met {what}: index {rec[1]}, value {rec[2]}, "
                                   f"limit {rec[3]}; it used page 0 instead, the step's results are not valid")

    def listed_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                         token_seq: torch.Tensor, slots: torch.Tensor, page_table: torch.Tensor,
                         block_list: torch.Tensor, n_kv: int, scale: float, tiles: bool = False) -> torch.Tensor:
        """Attention of every token over the 64-token key blocks its list names (block-sparse).  ``tiles``: the
        tokens are those of prompts (consecutive tokens mostly of one sequence); eight of them then share the
        blocks they bring from the cache."""
        self._act(q, "q")
        self._i32(block_list, "block list")
        n, n_heads, d = q.shape
        out = self.empty(n, n_heads * d)
        if (tiles and self.use_tcgen05_attention and self.use_tcgen05_listed and d == 128 and n_heads == 16 * n_kv
                and page_table.shape[1] <= self.lib.cpm_listed_attention_tcgen05_max_pages()):
            # prompt tokens of the long-context shape: eight tokens x sixteen heads are one tensor-core tile
            check(self.lib.cpm_listed_attention_tcgen05(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                                        _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                                        k_cache.shape[0], _ptr(block_list), block_list.shape[-1], n, n_heads,
                                                        n_kv, d, float(scale), self._stream()),
                  "block-list attention on tcgen05")
            return out
        n_splits = 1 if tiles else self.decode_splits(n, n_heads, n_kv)      # few tokens (decode): share a token's blocks out
        scratch = None
        if n_splits > 1:
            scratch = self.empty(self.lib.cpm_decode_attention_scratch_floats(n, n_heads, n_kv, d, n_splits),
                                 dtype=torch.float32)
        check(self.lib.cpm_listed_attention_bf16(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(positions),
                                                 _ptr(token_seq), _ptr(slots), _ptr(page_table), page_table.shape[1],
                                                 _ptr(block_list), block_list.shape[-1], n, n_heads, n_kv, d,
                                                 float(scale), _ptr(scratch), n_splits, 1 if tiles else 0, self._stream()),
              f"block-list attention (head_dim {d})")
        return out


LAUNCHES_EXTRA = library.LAUNCHES
