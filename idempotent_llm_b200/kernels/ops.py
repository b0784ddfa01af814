"""Python side of the CUDA kernels: shape checks, output allocation, the call.

``Kernels(dtype, device)`` loads the library compiled for that storage dtype
(``float32`` or ``bfloat16``) and exposes one method per kernel.  Every method
checks what the kernel cannot check itself and raises ``KernelError`` with the
library's message when a launch is refused.  There is no CPU path: constructing
``Kernels`` without a CUDA device raises.

Matrix products: the 32-bit library has its own FMA kernel (no tensor cores, no
reduced-precision mode).  In bfloat16 they run on the hand-written tcgen05
kernels of ``csrc/gemm_tcgen05.cu`` (the reference sends every matrix product to
a library, ``torch._int_mm``, src/detllm/backends.py:88-135).  No product is sent
to a library here, and none is split over its inner axis: an element is one chain
of additions whatever the step's size.

Environment switches (all default to the fast path): ``IDM_FUSED=0`` (epilogues as kernels of their
own), ``IDM_ATTENTION=generic`` (the general attention kernel for every step), ``IDM_PDL=0`` (no
programmatic dependent launch), ``IDM_PROGRAM=0`` (every kernel of a step called from Python instead
of one call that runs the step's list of calls).

The entry points are called through ctypes with declared argument types (``SIGNATURES``), so that a
call passes plain integers and floats; the current stream's handle comes from torch without a stream
object being built.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import builder

_DT = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


class KernelError(RuntimeError):
    pass


# the handle of the current stream of a device as an integer, without building a stream object
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# Every entry point of the libraries: result type and, per argument, p pointer (or stream) / i int /
# f float / q long long, in the order of the C declarations in csrc/ (a test reads the declarations
# and compares).
SIGNATURES = {
    "idm_last_error": (ctypes.c_char_p, ""),
    "idm_dtype_name": (ctypes.c_char_p, ""),
    "idm_page_tokens": (c_int, ""),
    "idm_set_pdl": (None, "i"),
    "idm_embed": (c_int, "pppiip"),
    "idm_embed_scaled": (c_int, "pppiifp"),
    "idm_post_pre_norm": (c_int, "pppfpfpiiip"),
    "idm_gated_act": (c_int, "ppiiip"),
    "idm_token_gate": (c_int, "pppiipiiip"),
    "idm_short_conv": (c_int, "piiiippipqppppppip"),
    "idm_conv_qkv_cache": (c_int, "piiippqiiiiipppppipppppip"),
    "idm_conv_state_update": (c_int, "piiiipqppppip"),
    "idm_ssd_chunk_tokens": (c_int, ""),
    "idm_ssd_scan": (c_int, "piiiipiiippppqpippiiiiippipip"),
    "idm_ssd_group_norm": (c_int, "piipffpiiip"),
    "idm_attention_sink": (c_int, "ppiifpppippipppppiiiiifip"),
    "idm_attention_biased": (c_int, "ppiifpppiipppiipppppiiiiififip"),
    "idm_head_finish": (c_int, "piiiipppppfipfiiiippppiipppip"),
    "idm_cols_cast": (c_int, "piiipiip"),
    "idm_delta_prep": (c_int, "piiipiipiiipppiiiip"),
    "idm_delta_scan": (c_int, "piiiipiippqpippiiiiiipp"),
    "idm_delta_scan_scratch_floats": (c_longlong, "iiii"),
    "idm_delta_out": (c_int, "pipfpiiifpiiiiip"),
    "idm_add_rmsnorm2": (c_int, "ppiqppfpppiip"),
    "idm_gemm_bf16_gated": (c_int, "pppiiiip"),
    "idm_add_rmsnorm": (c_int, "ppiqpfppiip"),
    "idm_rope_table": (c_int, "ppppiip"),
    "idm_qkv_finish": (c_int, "piqiiiippfpppppppiipppp"),
    "idm_kv_write_ring": (c_int, "pppppiippppiiip"),
    "idm_swiglu": (c_int, "piqpiiip"),
    "idm_sample_scratch_floats": (c_longlong, "ii"),
    "idm_sample": (c_int, "piifpppp"),
    "idm_decode_advance": (c_int, "pppppppiip"),
    "idm_attention_generic": (c_int, "pppppiipppppppiiiifip"),
    "idm_attention_decode_supports": (c_int, "i"),
    "idm_attention_decode_chunk": (c_int, ""),
    "idm_attention_decode_scratch_floats": (c_longlong, "iiii"),
    "idm_attention_decode": (c_int, "pppppiipppiiiiifip"),
    "idm_attention_decode_static": (c_int, "pppppiippiiiiifip"),
    "idm_attention_tc_supports": (c_int, "i"),
    "idm_attention_tc_heads_per_tile": (c_int, "ii"),
    "idm_attention_tc_scratch_floats": (c_longlong, "iiiiii"),
    "idm_attention_tc": (c_int, "ppppipippippppiiiifiiippiip"),
    "idm_attention_tc_sink": (c_int, "pppppipippippppiiiifiiippiip"),
    "idm_attention_tc_biased": (c_int, "ppppifippipippippppiiiifiiippiip"),
    "idm_gate_scale": (c_int, "ppiifpiiiip"),
    "idm_attention_tc_status": (c_int, ""),
    "idm_attention_tc_set_few_rows": (c_int, "i"),
    "idm_latent_kv_finish": (c_int, "piiiiipfpifppippppip"),
    "idm_headwise": (c_int, "pqiipipiqiiipifiip"),
    "idm_latent_attention_max_rank": (c_int, ""),
    "idm_latent_attention_heads_per_block": (c_int, "iii"),
    "idm_latent_attention": (c_int, "pppippppppiiiifiip"),
    "idm_latent_expand_pack": (c_int, "pippiiiiiipifippppipppip"),
    "idm_experts_few": (c_int, "pppppqqqpppiiiiiifp"),
    "idm_experts_major": (c_int, "pppppqqqppppiiiiiifp"),
    "idm_rows_gather": (c_int, "pppiip"),
    "idm_experts_grouped": (c_int, "ppipqpqppiiip"),
    "idm_experts_dense": (c_int, "ppppipqpqpppiiiiifp"),
    "idm_experts_grouped_step": (c_int, "pppppipqpqppppiiiiifp"),
    "idm_dense_ff": (c_int, "ppppppiiiip"),
    "idm_experts_combine": (c_int, "ppppiiifp"),
    "idm_route": (c_int, "pipppiiiiifp"),
    "idm_experts_identity": (c_int, "ppppiiiip"),
    "idm_post_layernorm": (c_int, "pppppfpiiip"),
    "idm_add_layernorm": (c_int, "ppiqppfppiip"),
    "idm_embed_bigram": (c_int, "ppppppppqppiiqqqp"),
    "idm_add_dyt": (c_int, "ppiqppfppiip"),
    "idm_act_cast": (c_int, "ppqip"),
    "idm_concat_cast": (c_int, "ppiqppiip"),
    "idm_logit_cap": (c_int, "pqffp"),
    "idm_gemm_f32": (c_int, "pppiiip"),
    "idm_gemm_set_small": (None, "iii"),
    "idm_gemm_set_small_max": (None, "i"),
    "idm_gemm_set_small_tiles": (None, "i"),
    "idm_gemm_set_wide_tiles": (None, "i"),
    "idm_gemm_set_pair": (None, "ii"),
    "idm_gemm_set_band_mb": (None, "i"),
    "idm_gemm_set_wide_from": (None, "i"),
    "idm_gemm_bf16": (c_int, "pppiiip"),
    "idm_gemm_bf16_residual": (c_int, "pppiiip"),
    "idm_gemm_bf16_swiglu": (c_int, "pppiiip"),
    "idm_gemm_bf16_qkv": (c_int, "ppiiiiippfppppppppiipppp"),
    "idm_gemm_status": (c_int, ""),
    "idm_wait_probe": (c_int, "qipp"),
    "idm_program_layout": (c_int, "p"),
    "idm_run_program": (c_int, "pipp"),
    # only in a library compiled with -DIDM_TRACE (time stamps from inside two kernels: a measuring aid)
    "idm_gemm_trace_read": (c_int, "p"),
    "idm_gemm_block_trace_read": (c_int, "p"),
    "idm_gemm_log_read": (c_int, "pi"),
    "idm_gemm_mma_trace_read": (c_int, "p"),
    "idm_attention_tc_trace_read": (c_int, "p"),
    "idm_attention_item_trace_read": (c_int, "pi"),
}


class Kernels:
    def __init__(self, dtype: torch.dtype, device):
        device = torch.device(device)
        if dtype not in _DT:
            raise KernelError(f"no kernels for dtype {dtype}; float32 and bfloat16 exist")
        if device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("the kernels run on a CUDA device only; there is no CPU path")
        cap = torch.cuda.get_device_capability(device)
        if cap[0] != 10:
            raise KernelError(f"the kernels are compiled for sm_100a; this device is sm_{cap[0]}{cap[1]}")
        self.dtype = dtype
        self.device = device
        self.lib = builder.load(_DT[dtype])
        self.launches = 0                     # kernels of this library launched so far
        self._scratch = {}
        self._padded_weights = {}
        self._single_tiles = {}
        self._device_index = device.index if device.index is not None else 0
        self._retired = []
        L = self.lib
        # argument and result types of every entry point: with them set, plain integers (addresses,
        # sizes), floats and None (a null pointer) go in as they are -- no ctypes object per argument
        kinds = {"p": c_void_p, "i": c_int, "f": c_float, "q": c_longlong}
        for name, (result, args) in SIGNATURES.items():
            fn = getattr(L, name, None)
            if fn is None:
                continue                      # an entry point of the other precision's library
            fn.restype = result
            fn.argtypes = [kinds[a] for a in args]
        # fused epilogues of the tensor-core product (residual add, SwiGLU, q/k/v finish): parts use
        # them when this is True and run separate kernels otherwise (IDM_FUSED=0, and the 32-bit library).
        # Which of the two runs never depends on how many tokens a step brings.
        self.fused = dtype == torch.bfloat16 and os.environ.get("IDM_FUSED", "1") != "0"
        # "tcgen05": attention on the tensor cores wherever that kernel has the head size (64, 128) and the
        # layer has no window; "general": the one-warp-per-query kernel everywhere.  Which kernel runs never
        # depends on the step's shape, so prompts and single tokens give the same bits.
        self.attention_impl = os.environ.get("IDM_ATTENTION", "tcgen05")
        # key blocks (of 64) of a run of the tensor-core kernel: each run starts its sums from nothing and
        # the runs are folded in ascending order, so this number is part of the arithmetic's definition
        self.attention_run_blocks = 8
        # prompts: tiles with more key blocks than a fair share are shared by several blocks; the pool holds that
        # many runs' results (of 128 rows x (head_dim + 2) floats)
        self.attention_share_tiles = True
        self.attention_share_scale, self.attention_share_min_runs = 1.0, 2
        self.attention_pool_slots = 4096
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.page = L.idm_page_tokens()
        # a model whose parts can emit their calls runs a step by one call into the library (program.py);
        # switched off (IDM_PROGRAM=0, or this attribute), every kernel is called from Python: the same bits
        self.use_programs = self.fused and os.environ.get("IDM_PROGRAM", "1") != "0"
        if hasattr(L, "idm_program_layout"):
            from . import program
            seen = (c_int * 16)()
            n = L.idm_program_layout(seen)
            if list(seen[:n]) != program.layout():
                raise KernelError(f"the records of a step program differ between the library {list(seen[:n])} "
                                  f"and the binding {program.layout()}")

    # ------------------------------------------------------------------ helpers
    def _stream(self):
        # (the stream object torch builds for current_stream() costs several microseconds per launch)
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, rc: int, n_launches: int = 1):
        if rc != 0:
            raise KernelError(self.lib.idm_last_error().decode())
        self.launches += n_launches

    def _need(self, t: torch.Tensor, dtype, what: str):
        if t.dtype != dtype or not t.is_cuda or not t.is_contiguous():
            raise KernelError(f"{what}: expected a contiguous CUDA tensor of {dtype}, got {t.dtype} "
                              f"{'cuda' if t.is_cuda else 'cpu'} contiguous={t.is_contiguous()}")

    def scratch(self, key: str, n_floats: int) -> torch.Tensor:
        """A 32-bit scratch buffer that only grows (its address is stable across steps once large enough)."""
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < n_floats:
            # a captured graph may still point at the old buffer: it is kept, never freed
            self._retired.append(buf)
            # zeros: kernels keep arrival counters in their scratch and leave them at zero
            buf = self._scratch[key] = torch.zeros(max(n_floats, 1), dtype=torch.float32, device=self.device)
        return buf

    # ------------------------------------------------------------------ kernels
    def embed(self, tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        self._need(tokens, torch.int32, "embed tokens")
        self._need(table, self.dtype, "embed table")
        n, hidden = tokens.numel(), table.shape[1]
        h = torch.empty((n, hidden), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_embed(_p(tokens), _p(table), _p(h),
                                       n, hidden, self._stream()))
        return h

    def embed_scaled(self, tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
        """``table[tokens] * scale`` as the 32-bit stream."""
        self._need(tokens, torch.int32, "embed tokens")
        self._need(table, self.dtype, "embed table")
        n, hidden = tokens.numel(), table.shape[1]
        h = torch.empty((n, hidden), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_embed_scaled(_p(tokens), _p(table), _p(h), n, hidden, float(scale), self._stream()))
        return h

    def post_pre_norm(self, h, y, w_post, eps: float, w_pre=None, eps_pre: float = 0.0, cast: bool = False):
        """``h += rmsnorm(y) * w_post`` in place; returns what the next sublayer reads: ``rmsnorm(h) * w_pre`` if
        ``w_pre`` is given, ``h`` in the storage dtype if ``cast``, else None."""
        self._need(h, torch.float32, "residual stream")
        self._need(y, torch.float32, "sublayer output")
        n, hidden = h.shape
        if tuple(y.shape) != (n, hidden) or w_post.numel() != hidden or (w_pre is not None and w_pre.numel() != hidden):
            raise KernelError(f"post_pre_norm: stream {tuple(h.shape)}, output {tuple(y.shape)}, weights {w_post.numel()}")
        mode = 1 if w_pre is not None else 2 if cast else 0
        x = torch.empty((n, hidden), dtype=self.dtype, device=self.device) if mode else None
        self._check(self.lib.idm_post_pre_norm(_p(h), _p(y), _p(w_post), eps, _p(w_pre), eps_pre, _p(x), mode, n,
                                               hidden, self._stream()))
        return x

    def gated_act(self, gu: torch.Tensor, act: int) -> torch.Tensor:
        """``act(gate) * up`` of a 32-bit gate/up product ``[N, 2 * inter]`` (gate columns, then up columns);
        ``act``: 0 silu, 1 gelu (tanh form)."""
        self._need(gu, torch.float32, "gate-up")
        n, width = gu.shape
        y = torch.empty((n, width // 2), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_gated_act(_p(gu), _p(y), n, width // 2, act, self._stream()))
        return y

    def token_gate(self, s, tokens, table, col0: int, act: int) -> torch.Tensor:
        """``act(s[t]) * table[tokens[t], col0 : col0 + dim]`` in the storage dtype ``[N, dim]``."""
        self._need(s, torch.float32, "token gate input")
        self._need(table, self.dtype, "token table")
        n, dim = s.shape
        y = torch.empty((n, dim), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_token_gate(_p(s), _p(tokens), _p(table), table.shape[1], col0, _p(y), n, dim, act,
                                            self._stream()))
        return y

    @staticmethod
    def _state_stride(state: Optional[torch.Tensor]) -> int:
        """Floats between two slots' regions of a per-sequence state ``[max_seqs, n]`` (a view of a wider one)."""
        if state is None:
            return 0
        if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1:
            raise KernelError("per-sequence state must be a 32-bit [slots, n] view with unit inner stride")
        return state.stride(0)

    def short_conv(self, proj, col0: int, channels: int, w, bias, act: int, state, ctx) -> torch.Tensor:
        """Causal filter over time of columns ``[col0, col0 + channels)`` of the 32-bit ``proj [N, width]``; returns
        32-bit ``[N, channels]``.  ``state [slots, (taps - 1) * channels]`` holds each sequence's last inputs."""
        self._need(proj, torch.float32, "projection")
        n, width = proj.shape
        taps = w.shape[1]
        out = torch.empty((n, channels), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_short_conv(_p(proj), width, col0, channels, taps, _p(w), _p(bias), act, _p(state),
                                            self._state_stride(state), _p(out), _p(ctx.token_seq), _p(ctx.positions),
                                            _p(ctx.slots), _p(ctx.q_start), _p(ctx.cu_q), n, self._stream()))
        return out

    def conv_qkv_cache(self, proj, col0: int, w, state, n_q, n_kv, dk, dv, cs, kv, ctx) -> torch.Tensor:
        """q, k, v channels of ``proj`` filtered, q and k turned by the rotary table ``cs [N, half, 2]`` (or None),
        k and v written to the cache entry; returns q ``[N, n_q, dk]``."""
        self._need(proj, torch.float32, "projection")
        n, width = proj.shape
        half = 0 if cs is None else cs.shape[1]
        if cs is not None and (cs.shape[0] != n or cs.dtype != torch.float32):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {n} tokens")
        self._check_kv(kv, n_kv, dk, dv)
        q = torch.empty((n, n_q, dk), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_conv_qkv_cache(_p(proj), width, col0, w.shape[1], _p(w), _p(state),
                                                self._state_stride(state), n_q, n_kv, dk, dv, half, _p(cs), _p(q),
                                                _p(kv.k), _p(kv.v), _p(kv.table), kv.table.shape[1],
                                                _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), _p(ctx.q_start),
                                                _p(ctx.cu_q), n, self._stream()))
        return q

    def conv_state_update(self, proj, col0: int, channels: int, taps: int, state, ctx) -> None:
        """After a step of several tokens per sequence: the filter's state becomes each sequence's last inputs."""
        if taps <= 1:
            return
        self._check(self.lib.idm_conv_state_update(_p(proj), proj.shape[1], col0, channels, taps, _p(state),
                                                   self._state_stride(state), _p(ctx.slots), _p(ctx.q_start),
                                                   _p(ctx.cu_q), _p(ctx.kv_len), ctx.n_seqs, self._stream()))

    def ssd_chunks(self, ctx):
        """How a step's long portions are cut for the state-space recurrence: (chunk borders in packed tokens
        [n_chunks + 1], each sequence's first chunk [n_seqs + 1], n_chunks), on the device, made once a step; None
        when no sequence brings more than a chunk's tokens (then every sequence runs token by token from its state)."""
        L = self.lib.idm_ssd_chunk_tokens()
        if ctx.single_token or ctx.max_q_len <= L:
            return None
        plan = ctx.memo.get("ssd_chunks")
        if plan is None:
            borders, first, at = [], [0], 0
            for n in ctx.host_q_lens:
                borders += list(range(at, at + n, L))
                at += n
                first.append(len(borders))
            borders.append(at)
            dev = torch.tensor(borders + first, dtype=torch.int32).to(self.device)
            plan = ctx.memo["ssd_chunks"] = (dev, dev[:len(borders)], dev[len(borders):], len(borders) - 1)
        return plan

    def ssd_scan(self, xbc, cols, proj, z_col: int, dt_col: int, dt_bias, a_log, d_skip, state, ctx, heads, groups,
                 P, N) -> torch.Tensor:
        """The state-space recurrence over the step's tokens, sequence by sequence; returns the gated output
        ``y * silu(z)`` in 32-bit ``[N_tok, heads * P]`` and moves ``state [slots, heads * N * P]`` on.  Steps with
        long portions run them in chunks side by side (``ssd_chunks``)."""
        self._need(xbc, torch.float32, "filtered projection")
        self._need(proj, torch.float32, "projection")
        n = xbc.shape[0]
        y = torch.empty((n, heads * P), dtype=torch.float32, device=self.device)
        plan = self.ssd_chunks(ctx)
        chunk_t0 = seq_chunk0 = scratch = None
        n_chunks = 0
        if plan is not None:
            _, chunk_t0, seq_chunk0, n_chunks = plan
            scratch = self.scratch("ssd_scan", n_chunks * heads * N * P + n * heads)
        self._check(self.lib.idm_ssd_scan(_p(xbc), xbc.shape[1], cols[0], cols[1], cols[2], _p(proj), proj.shape[1],
                                          z_col, dt_col, _p(dt_bias), _p(a_log), _p(d_skip), _p(state),
                                          self._state_stride(state), _p(y), heads * P, _p(ctx.cu_q), _p(ctx.slots),
                                          ctx.n_seqs, heads, groups, P, N, _p(chunk_t0), _p(seq_chunk0), n_chunks,
                                          _p(scratch), n, self._stream()), 3 if n_chunks else 1)
        return y

    def ssd_group_norm(self, y, parts: int, w, eps: float, scale: float, out, out_col: int) -> None:
        """``out[:, out_col : out_col + width] = rmsnorm over each of `parts` equal parts of y * w * scale``."""
        self._need(y, torch.float32, "gated output")
        self._need(out, self.dtype, "norm output")
        n, width = y.shape
        self._check(self.lib.idm_ssd_group_norm(_p(y), width, parts, _p(w), eps, float(scale), _p(out), out.shape[1],
                                                out_col, n, self._stream()))

    def attention_sink(self, q, kv, ctx, scale: float, sink, gate, gate_stride: int, out, out_col: int,
                       out_scale: float) -> None:
        """Causal attention over the cache entry with a sink per head (or None) and a sigmoid gate (a 32-bit view
        ``[N, n_q * dv]`` with row stride ``gate_stride``, or None); the result times ``out_scale`` goes to
        ``out[:, out_col : out_col + n_q * dv]``."""
        self._need(q, self.dtype, "q")
        self._need(out, self.dtype, "attention output")
        n, n_q, dk = q.shape
        dv = kv.v_head_dim
        self._check_kv(kv, kv.n_kv_heads, dk, dv)
        self._check(self.lib.idm_attention_sink(
            _p(q), _p(out), out.shape[1], out_col, float(out_scale), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], _p(sink), (gate.data_ptr() if gate is not None else None), gate_stride,
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), _p(ctx.q_start), _p(ctx.cu_q), n, n_q,
            kv.n_kv_heads, dk, dv, scale, 0, self._stream()))

    def attention_biased(self, q, kv, ctx, scale: float, out, out_col: int, out_scale: float = 1.0, sink=None,
                         slopes=None, gate=None, gate_stride: int = 0, gate_per_head: bool = False, window=None,
                         softcap: float = 0.0, keep_first: int = 0) -> None:
        """The general attention kernel with all of its options: ``sink`` [n_q] joins the denominator, ``slopes`` [n_q]
        times the distance to a key is taken off its score, ``window`` keys are seen (and, whatever the distance, the
        sequence's first ``keep_first``), scores are capped at ``softcap * tanh(score / softcap)``, the result is multiplied by
        ``sigmoid(gate)`` (one number per head at ``gate[t, head]`` or one per channel) and by ``out_scale`` and
        stored at columns ``out_col ..`` of ``out``."""
        n, n_q, dk = q.shape
        self._check_kv(kv, kv.n_kv_heads, dk, kv.v_head_dim)
        for name, t in (("sink", sink), ("slopes", slopes)):
            if t is not None and (t.dtype != torch.float32 or t.numel() != n_q):
                raise KernelError(f"attention: {name} must hold one 32-bit number per head")
        self._check(self.lib.idm_attention_biased(
            _p(q), _p(out), out.shape[1], out_col, float(out_scale), _p(kv.k), _p(kv.v), _p(kv.table), kv.table.shape[1],
            kv.ring, _p(sink), _p(slopes), _p(gate), gate_stride, 1 if gate_per_head else 0, _p(ctx.token_seq),
            _p(ctx.positions), _p(ctx.slots), _p(ctx.q_start), _p(ctx.cu_q), n, n_q, kv.n_kv_heads, dk, kv.v_head_dim,
            float(scale), int(window) if window else 0, float(softcap or 0.0), int(keep_first or 0), self._stream()))

    def head_finish(self, proj, col_q: int, col_k: int, col_v, n_q: int, n_kv: int, dk: int, dv: int, biases, gammas,
                    eps: float, cs, mag: float, kv, ctx) -> torch.Tensor:
        """Bias, norm per head and partial rotation of the q and k heads in columns of the 32-bit ``proj``; k and v to
        the cache entry (``col_v`` None: the keys as projected are the values); returns q ``[N, n_q, dk]``."""
        self._need(proj, torch.float32, "projection")
        n, width = proj.shape
        self._check_kv(kv, n_kv, dk, dv)
        half = 0 if cs is None else cs.shape[1]
        if cs is not None and (cs.dtype != torch.float32 or tuple(cs.shape) != (n, half, 2)):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {(n, half, 2)}")
        bq, bk, bv = biases
        gq, gk = gammas
        q = torch.empty((n, n_q, dk), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_head_finish(
            _p(proj), width, col_q, col_k, -1 if col_v is None else col_v, _p(bq), _p(bk), _p(bv), _p(gq), _p(gk),
            float(eps), half, _p(cs), float(mag), n_q, n_kv, dk, dv, _p(q), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), n, self._stream()))
        return q

    def cols_cast(self, proj, col0: int, width: int, out_width: int) -> torch.Tensor:
        """Columns ``[col0, col0 + width)`` of a 32-bit buffer as a matrix operand ``[N, out_width]`` in the storage
        type, zero beyond ``width``."""
        self._need(proj, torch.float32, "projection")
        n = proj.shape[0]
        out = torch.empty((n, out_width), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_cols_cast(_p(proj), proj.shape[1], col0, width, _p(out), out_width, n, self._stream()))
        return out

    def delta_prep(self, c, c_q: int, c_k: int, a, a_col: int, proj, b_col: int, dt_bias, a_log, H: int, Hk: int,
                   dk: int, head_col: int = -1) -> torch.Tensor:
        """In place: q and k heads of ``c`` become unit vectors (q times ``dk ** -0.5``), columns ``a_col ..`` of ``a``
        become decays (``head_col`` >= 0: one decay per head from ``proj[:, head_col + h]``, written to all of the head's
        columns of ``a``); returns ``beta [N, H]``."""
        n = c.shape[0]
        beta = torch.empty((n, H), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_delta_prep(_p(c), c.shape[1], c_q, c_k, _p(a), a.shape[1], a_col, _p(proj), proj.shape[1],
                                            b_col, int(head_col), _p(dt_bias), _p(a_log), _p(beta), H, Hk, dk, n, self._stream()))
        return beta

    def delta_scan(self, c, c_q: int, c_k: int, c_v: int, g, g_col: int, beta, state, ctx, H: int, Hk: int, dk: int,
                   dv: int) -> torch.Tensor:
        """The gated delta rule over the step's tokens from and to each sequence's state ``[slots, H * dv * dk]``;
        returns the read-outs ``[N, H * dv]`` in 32-bit."""
        n = c.shape[0]
        o = torch.empty((n, H * dv), dtype=torch.float32, device=self.device)
        want = int(self.lib.idm_delta_scan_scratch_floats(n, H, dk, int(ctx.max_q_len)))
        scratch = torch.empty((want,), dtype=torch.float32, device=self.device) if want else None
        self._check(self.lib.idm_delta_scan(_p(c), c.shape[1], c_q, c_k, c_v, _p(g), g.shape[1], g_col, _p(beta), _p(state),
                                            self._state_stride(state), _p(o), H * dv, _p(ctx.cu_q), _p(ctx.slots),
                                            ctx.n_seqs, H, Hk, dk, dv, int(ctx.max_q_len), _p(scratch), self._stream()))
        return o

    def delta_out(self, o, w, eps: float, gate, gate_col: int, scale: float, out, out_col: int, H: int, dv: int,
                  gate_act: int = 0) -> None:
        """``out[:, out_col ..] = rmsnorm over each head of o * w * act(gate columns) * scale``; ``gate_act`` 0: sigmoid,
        1: silu."""
        n = o.shape[0]
        self._check(self.lib.idm_delta_out(_p(o), o.shape[1], _p(w), float(eps), _p(gate), gate.shape[1], gate_col,
                                           int(gate_act), float(scale), _p(out), out.shape[1], out_col, n, H, dv, self._stream()))

    def add_rmsnorm2(self, h, delta, gamma1, gamma2, eps: float, post=None):
        """``h += delta`` in place, then both norms of the same row from one root mean square: returns ``(norm(h) *
        gamma1, norm(h) * gamma2)`` (the second None without ``gamma2``); ``post`` [hidden] is added to the stream
        after the norms were taken."""
        self._need(h, torch.float32, "residual stream")
        n, hidden = h.shape
        P, stride = 0, 0
        if delta is not None:
            self._need(delta, torch.float32, "delta")
            if delta.dim() != 3 or tuple(delta.shape[1:]) != (n, hidden):
                raise KernelError(f"delta {tuple(delta.shape)} does not match the stream {(n, hidden)}")
            P, stride = delta.shape[0], n * hidden
        x1 = torch.empty((n, hidden), dtype=self.dtype, device=self.device)
        x2 = torch.empty((n, hidden), dtype=self.dtype, device=self.device) if gamma2 is not None else None
        self._check(self.lib.idm_add_rmsnorm2(_p(h), _p(delta), P, stride, _p(gamma1), _p(gamma2), float(eps), _p(x1),
                                              _p(x2), _p(post), n, hidden, self._stream()))
        return x1, x2

    def gemm_gated(self, x, w_tiled, inter: int, act: int) -> torch.Tensor:
        """``act(x . gate^T) * (x . up^T)`` in the storage dtype ``[M, inter]`` (``tile_gate_up`` layout)."""
        M, N, Kd = self._gemm_shape(x, w_tiled)
        if N != -(-inter // 64) * 128:
            raise KernelError(f"tiled gate/up weight has {N} rows, expected {-(-inter // 64) * 128}")
        y = torch.empty((M, inter), dtype=self.dtype, device=self.device)
        if M:
            self._check(self.lib.idm_gemm_bf16_gated(_p(x), _p(w_tiled), _p(y), M, inter, Kd, act, self._stream()))
        return y

    def add_rmsnorm(self, h, delta, gamma, eps: float, rows=None) -> torch.Tensor:
        self._need(h, torch.float32, "residual stream")
        self._need(gamma, torch.float32, "norm weight")
        n, hidden = h.shape
        if gamma.numel() != hidden:
            raise KernelError(f"norm weight has {gamma.numel()} elements, rows have {hidden}")
        P, stride = 0, 0
        if delta is not None:
            self._need(delta, torch.float32, "delta")
            if delta.dim() != 3 or tuple(delta.shape[1:]) != (n, hidden):
                raise KernelError(f"delta {tuple(delta.shape)} does not match the stream {(n, hidden)}")
            P, stride = delta.shape[0], n * hidden
        if rows is not None:
            self._need(rows, torch.int32, "rows")
        n_out = n if rows is None else rows.numel()
        x = torch.empty((n_out, hidden), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_add_rmsnorm(_p(h), _p(delta), P, stride,
                                             _p(gamma), eps, _p(x),
                                             _p(rows), n_out, hidden, self._stream()))
        return x

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        self._need(positions, torch.int32, "positions")
        self._need(inv_freq, torch.float64, "inv_freq")
        n, half = positions.numel(), inv_freq.numel()
        cs = torch.empty((n, half, 2), dtype=torch.float32, device=self.device)
        # for steps of many tokens also as [half, n, 2]: the q/k/v product's epilogue of such steps has
        # a thread per token and reads the tokens of one dim side by side
        by_dim = torch.empty((half, n, 2), dtype=torch.float32, device=self.device) if n > 64 else None
        self._check(self.lib.idm_rope_table(_p(positions), _p(inv_freq), _p(cs), _p(by_dim),
                                            n, half, self._stream()))
        cs.by_dim = by_dim
        return cs

    def qkv_finish(self, qkv, n_q, n_kv, hd, q_gamma, k_gamma, eps, cs, ctx, kv, keep_new: bool):
        """Norm + rotation of q and k heads; k, v to the cache entry ``kv`` (if given) and/or to packed
        buffers (``keep_new``).  Returns (q [N, n_q, hd], k_new, v_new)."""
        self._need(qkv, torch.float32, "qkv")
        P, n, width = qkv.shape
        if width != (n_q + 2 * n_kv) * hd:
            raise KernelError(f"qkv rows have {width} elements, expected {(n_q + 2 * n_kv) * hd}")
        if cs is not None and tuple(cs.shape) != (n, hd // 2, 2):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {(n, hd // 2, 2)}")
        for gmm in (q_gamma, k_gamma):
            if gmm is not None and gmm.numel() != hd:
                raise KernelError("q/k norm weight must have head_dim elements")
        q = torch.empty((n, n_q, hd), dtype=self.dtype, device=self.device)
        k_new = v_new = None
        if keep_new and n_kv:
            k_new = torch.empty((n, n_kv, hd), dtype=self.dtype, device=self.device)
            v_new = torch.empty((n, n_kv, hd), dtype=self.dtype, device=self.device)
        if kv is not None:
            self._check_kv(kv, n_kv, hd)
        self._check(self.lib.idm_qkv_finish(
            _p(qkv), P, n * width, n, n_q, n_kv, hd,
            _p(q_gamma), _p(k_gamma), eps, _p(cs),
            _p(q), _p(k_new), _p(v_new),
            (_p(kv.k) if kv is not None else None), (_p(kv.v) if kv is not None else None),
            (_p(kv.table) if kv is not None else None),
            (kv.table.shape[1] if kv is not None else 0), (kv.ring if kv is not None else 0),
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), self._stream()))
        return q, k_new, v_new

    def _check_kv(self, kv, n_kv, hd, v_hd=None):
        if kv.k.dtype != self.dtype or kv.k.shape[1:] != (n_kv, self.page, hd) or not kv.k.is_contiguous():
            raise KernelError(f"cache entry {tuple(kv.k.shape)} {kv.k.dtype} does not fit "
                              f"[pages, {n_kv}, {self.page}, {hd}] {self.dtype}")
        v_hd = hd if v_hd is None else v_hd
        if kv.v.dtype != self.dtype or kv.v.shape[1:] != (n_kv, self.page, v_hd) or not kv.v.is_contiguous():
            raise KernelError(f"cache entry's values {tuple(kv.v.shape)} {kv.v.dtype} do not fit "
                              f"[pages, {n_kv}, {self.page}, {v_hd}] {self.dtype}")

    def kv_write_ring(self, k_new, v_new, kv, ctx) -> None:
        n, n_kv, hd = k_new.shape
        self._check_kv(kv, n_kv, hd)
        self._check(self.lib.idm_kv_write_ring(
            _p(k_new), _p(v_new), _p(kv.k), _p(kv.v),
            _p(kv.table), kv.table.shape[1], kv.ring, _p(ctx.token_seq),
            _p(ctx.positions), _p(ctx.slots), _p(ctx.kv_len), n,
            n_kv, hd, self._stream()))

    def attention(self, q, kv, ctx, k_new, v_new, scale: float, window) -> torch.Tensor:
        """Causal attention of the step's queries over the cache entry; returns [N, n_q * hd].

        One kernel per (dtype, head size, window or not) whatever the step looks like: the 32-bit
        library and windowed layers take the general kernel, bfloat16 with head sizes 64 and 128 the
        tensor-core kernel, for prompts and for single tokens alike."""
        self._need(q, self.dtype, "q")
        n, n_q, hd = q.shape
        self._check_kv(kv, kv.n_kv_heads, hd)
        w = int(window) if window else 0
        if (self.dtype == torch.bfloat16 and self.attention_impl == "tcgen05" and k_new is None and not w
                and kv.ring == 0 and self.lib.idm_attention_tc_supports(hd)):
            return self.attention_tc(q, kv, ctx, scale)
        return self.attention_generic(q, kv, ctx, k_new, v_new, scale, window)

    def attention_tc(self, q, kv, ctx, scale: float, out=None, through_scratch=None, share=None, sink=None, slopes=None,
                     window=None, softcap: float = 0.0, keep_first: int = 0) -> torch.Tensor:
        """Causal attention on the tensor cores: tiles of (128 / gp tokens) x (gp q-heads of one kv-head).

        Steps with few tokens per sequence (at most 32 rows a tile: single tokens above all) give every
        run of key blocks a block of its own, and the runs meet in scratch; other steps let one block
        walk a tile's runs, except that tiles with more key blocks than a fair share of the step's are
        shared by several blocks.  ``through_scratch`` and ``share`` force one way or the other (tests: the
        bits are the same)."""
        n, n_q, hd = q.shape
        if out is None:
            out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        (tile_seq, tile_start, n_tiles, rows_cap, max_runs, scratch, tile_pool, max_parts,
         per) = self.attention_tc_plan(ctx, n_q, kv.n_kv_heads, hd, through_scratch, share)
        rest = (_p(kv.k), _p(kv.v), kv.k.shape[0],
                _p(kv.table), kv.table.shape[1], tile_seq, tile_start, n_tiles, _p(ctx.cu_q), _p(ctx.q_start),
                _p(ctx.kv_len), _p(ctx.slots), n, n_q, kv.n_kv_heads,
                hd, scale, self.attention_run_blocks, max_runs, rows_cap, scratch, tile_pool, max_parts, per,
                self._stream())
        if slopes is not None or window or softcap:
            # a slope per q-head times the distance to a key off its score, and a window of keys a query sees (runs of
            # key blocks before every window of a tile are not walked)
            for name, t in (("sink", sink), ("slopes", slopes)):
                if t is not None and (t.dtype != torch.float32 or t.numel() != n_q):
                    raise KernelError(f"attention: {name} must hold one 32-bit number per head")
            self._check(self.lib.idm_attention_tc_biased(_p(q), _p(out), _p(sink), _p(slopes), int(window) if window else 0,
                                                         float(softcap or 0.0), int(keep_first or 0), *rest))
        elif sink is None:
            self._check(self.lib.idm_attention_tc(_p(q), _p(out), *rest))
        else:
            # a learned score per q-head that joins the softmax's sum with no key and no value
            self._need(sink, torch.float32, "sink")
            if sink.numel() != n_q:
                raise KernelError(f"{sink.numel()} sinks for {n_q} q-heads")
            self._check(self.lib.idm_attention_tc_sink(_p(q), _p(out), _p(sink), *rest))
        return out

    def attention_tc_fits(self, kv, hd: int, dv: int) -> bool:
        """Whether the tensor-core attention has this layer: bfloat16, key and value rows of one width that it has
        a kernel for, no ring."""
        return (self.dtype == torch.bfloat16 and self.attention_impl == "tcgen05" and hd == dv and kv.ring == 0
                and bool(self.lib.idm_attention_tc_supports(hd)))

    def gate_scale(self, o, gate, gate_stride: int, scale: float, out, out_col: int, gate_group: int = 1) -> None:
        """``out[:, out_col : out_col + width] = o * sigmoid(gate) * scale`` (``gate``: a 32-bit view with row stride
        ``gate_stride``, or None for the constant alone; ``gate_group`` columns in a row share one gate number: a head's
        size for a gate per head)."""
        self._need(o, self.dtype, "mixer output")
        self._need(out, self.dtype, "gated output")
        n, width = o.shape
        self._check(self.lib.idm_gate_scale(_p(o), (gate.data_ptr() if gate is not None else None), gate_stride, int(gate_group),
                                            float(scale), _p(out), out.shape[1], out_col, n, width, self._stream()))

    def attention_tc_plan(self, ctx, n_q: int, n_kv: int, hd: int, through_scratch=None, share=None):
        """What the attention launches of one step share, for one arrangement of heads: the list of tiles
        (on the device; made once a step), how the tiles' runs are spread over blocks, and the scratch.
        Returns (tile_seq, tile_start, n_tiles, rows_cap, max_runs, scratch, tile_pool, max_parts,
        runs_per_part) as ``idm_attention_tc`` takes them (addresses as integers or None)."""
        gp = self.lib.idm_attention_tc_heads_per_tile(n_q, n_kv)
        tok = 128 // gp
        R = self.attention_run_blocks
        # (the spread of shared tiles over the pool depends on the number of head groups: layers with other head counts
        # have plans of their own)
        memo_key = ("attention_tc_tiles", gp, n_q // gp)
        tiles = ctx.memo.get(memo_key)
        if tiles is None and ctx.single_token:
            # one tile per sequence: the same list for every step of that many sequences (kept, so that a
            # step being captured into a graph copies nothing from the host)
            tiles = self._single_tiles.get((ctx.n_seqs, gp))
            if tiles is None:
                dev = torch.stack([torch.arange(ctx.n_seqs, dtype=torch.int32),
                                   torch.zeros(ctx.n_seqs, dtype=torch.int32)]).to(self.device)
                tiles = self._single_tiles[(ctx.n_seqs, gp)] = (dev, dev[0].data_ptr(), dev[1].data_ptr(), ctx.n_seqs, gp)
        if tiles is None:
            # (sequence, first token of the tile); tiles with the most keys first, so that the longest
            # blocks start first
            items = []
            for i, L in enumerate(ctx.host_q_lens):
                for st in range(0, L, tok):
                    items.append((ctx.host_starts[i] + min(st + tok - 1, L - 1), i, st))
            items.sort(key=lambda t: -t[0])
            rows_cap = min(tok, max(ctx.host_q_lens)) * gp
            # Tiles with more key blocks than a fair share of the step's are shared by several blocks, each
            # walking `per` runs and leaving every run's result in a pool; the last block to arrive folds them
            # in the order of the runs (the same bits as one block walking them all: the runs are the same).
            n_hg = n_q // gp
            blocks_of = [last // self.page + 1 for last, _, _ in items]
            fair = -(-int(sum(blocks_of) * n_hg * self.attention_share_scale) // (2 * self.sm_count))
            per = max(self.attention_share_min_runs, -(-fair // R))   # runs a block walks
            pool, slots_used, max_parts = [], 0, 1
            for nb in blocks_of:
                runs = -(-nb // R)
                if self.attention_share_tiles and rows_cap == 128 and runs > per and slots_used + runs * n_hg <= self.attention_pool_slots:
                    pool.append(slots_used)
                    slots_used += runs * n_hg
                    max_parts = max(max_parts, -(-runs // per))
                else:
                    pool.append(-1)
            host = torch.tensor([[i for _, i, _ in items], [st for _, _, st in items], pool], dtype=torch.int32)
            dev = host.to(self.device)
            plan = (dev[2].data_ptr(), max_parts, per, slots_used) if slots_used else (None, 0, 0, 0)
            tiles = ctx.memo[memo_key] = (dev, dev[0].data_ptr(), dev[1].data_ptr(), len(items), rows_cap, plan)
        _, tile_seq, tile_start, n_tiles, rows_cap = tiles[:5]
        tile_pool, max_parts, per, pool_slots = tiles[5] if len(tiles) > 5 else (None, 0, 0, 0)
        # an upper bound of the key blocks any tile has (a captured step is replayed at growing lengths)
        longest = -(-ctx.max_kv_len // self.page)
        max_runs = -(-longest // R)
        if through_scratch is None:
            # every run a block of its own where a tile has few rows (single tokens above all): the runs'
            # results are small then.  For whole tiles of a prompt the way through scratch was measured
            # slower (2048 tokens: 88 us against 45 us), although it spreads a long tile over several blocks.
            through_scratch = rows_cap <= 32
        if through_scratch:
            need = self.lib.idm_attention_tc_scratch_floats(n_tiles, n_q, n_kv, hd, max_runs, rows_cap)
            tile_pool, max_parts, per = None, 0, 0
        else:
            if share is False:
                tile_pool, max_parts, per, pool_slots = None, 0, 0, 0
            need = self.lib.idm_attention_tc_scratch_floats(n_tiles, n_q, n_kv, hd, 0, 0) if (max_runs > 1 or pool_slots) else 0
            need += pool_slots * (-(-(128 * (hd + 2)) // 4) * 4)
            max_runs = 0
        scratch = self.scratch("attention_tc", need) if need else None
        return tile_seq, tile_start, n_tiles, rows_cap, max_runs, _p(scratch), tile_pool, max_parts, per

    def attention_tc_few_rows(self, on: bool) -> bool:
        """Whether tiles of at most 16 rows take the kernel made for them (the default) or the one all
        other tiles take; returns the old setting.  Tests compare the two bit for bit."""
        return bool(self.lib.idm_attention_tc_set_few_rows(1 if on else 0))

    def attention_tc_status(self) -> int:
        """Non-zero if a bounded wait inside an attention kernel ran out since the last call (the result
        of that launch is wrong).  The kernels' counters in scratch may then be left standing, so the
        scratch is cleared."""
        if self.dtype == torch.float32:
            return 0
        status = self.lib.idm_attention_tc_status()
        if status and "attention_tc" in self._scratch:
            self._scratch["attention_tc"].zero_()
        return status

    def attention_generic(self, q, kv, ctx, k_new, v_new, scale: float, window) -> torch.Tensor:
        """The general kernel, whatever the step's shape (tests compare the special kernels with it)."""
        n, n_q, hd = q.shape
        out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_attention_generic(
            _p(q), _p(out), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(k_new), _p(v_new),
            _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots),
            _p(ctx.q_start), _p(ctx.cu_q), n, n_q, kv.n_kv_heads,
            hd, scale, (int(window) if window else 0), self._stream()))
        return out

    def attention_decode(self, q, kv, slots, kv_len, max_kv_len: int, scale: float, window: int,
                         out=None) -> torch.Tensor:
        """One query per sequence against its cached keys (split over chunks of keys, then merged)."""
        n, n_q, hd = q.shape
        if out is None:
            out = torch.empty((n, n_q * hd), dtype=self.dtype, device=self.device)
        n_chunks = -(-max_kv_len // self.lib.idm_attention_decode_chunk())
        need = self.lib.idm_attention_decode_scratch_floats(n, n_q, n_chunks, hd)
        scratch = self.scratch("attention_decode", need)
        self._check(self.lib.idm_attention_decode(
            _p(q), _p(out), _p(kv.k), _p(kv.v), _p(kv.table),
            kv.table.shape[1], kv.ring, _p(slots), _p(kv_len),
            _p(scratch), n, n_q, kv.n_kv_heads, hd, max_kv_len,
            scale, window, self._stream()))
        return out

    def swiglu(self, gu: torch.Tensor, tiled_inter: Optional[int] = None) -> torch.Tensor:
        """``g * sigmoid(g) * u`` of the gate/up product ``[P, N, 2 * inter]`` (gate columns, then up
        columns), or of its tiled form ``[P, N, ceil(inter / 64) * 128]`` when ``tiled_inter`` is given."""
        self._need(gu, torch.float32, "gate-up")
        P, n, width = gu.shape
        if tiled_inter is None:
            if width % 2:
                raise KernelError("gate-up rows must have an even number of elements")
            inter, tiled = width // 2, 0
        else:
            inter, tiled = int(tiled_inter), 1
            if width != -(-inter // 64) * 128:
                raise KernelError(f"tiled gate-up rows have {width} elements, expected {-(-inter // 64) * 128}")
        y = torch.empty((n, inter), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_swiglu(_p(gu), P, n * width, _p(y),
                                        n, inter, tiled, self._stream()))
        return y

    def gemm(self, x: torch.Tensor, w: torch.Tensor, pad: bool = False) -> torch.Tensor:
        """``x [M, K] . w [N, K]^T`` in 32-bit as ``[1, M, N]`` (the leading axis is the one a part's
        delta carries: partial sums that the consumer adds; these kernels never split a sum)."""
        return self.gemm_store(x, w, pad=pad).unsqueeze(0)

    def _gemm_shape(self, x, w):
        self._need(x, self.dtype, "gemm input")
        self._need(w, self.dtype, "gemm weight")
        M, Kd = x.shape
        N, K2 = w.shape
        if Kd != K2:
            raise KernelError(f"gemm: input rows have {Kd} elements, weight rows {K2}")
        if self.dtype == torch.bfloat16 and Kd % 8:
            raise KernelError(f"gemm: the inner size {Kd} must be a multiple of 8 in bfloat16 (rows on 16-byte borders)")
        return M, N, Kd

    def _padded(self, x, w):
        """bfloat16 operands whose inner size is no multiple of 8 (rows would not start on 16-byte borders), with zero
        columns added to both: the product is the same sum.  The padded matrix is made once and kept."""
        pad = -x.shape[1] % 8
        if self.dtype != torch.bfloat16 or not pad:
            return x, w
        key = (w.data_ptr(), tuple(w.shape))
        wp = self._padded_weights.get(key)
        if wp is None:
            wp = torch.zeros((w.shape[0], w.shape[1] + pad), dtype=w.dtype, device=w.device)
            wp[:, :w.shape[1]] = w
            self._padded_weights[key] = wp
        xp = torch.zeros((x.shape[0], x.shape[1] + pad), dtype=x.dtype, device=x.device)
        xp[:, :x.shape[1]] = x
        return xp, wp

    def gemm_store(self, x, w, pad: bool = False, out=None) -> torch.Tensor:
        """``x . w^T`` in 32-bit ``[M, N]``.  ``pad``: a bfloat16 inner size that is no multiple of 8 is served with
        zero columns added to both operands instead of being refused.  ``out``: a contiguous 32-bit ``[M, N]`` to write."""
        if pad:
            x, w = self._padded(x, w)
        M, N, Kd = self._gemm_shape(x, w)
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=self.device)
        else:
            self._need(out, torch.float32, "gemm output")
            if tuple(out.shape) != (M, N):
                raise KernelError(f"gemm: output {tuple(out.shape)} does not match the product {(M, N)}")
        if M:
            if self.dtype == torch.float32:
                self._check(self.lib.idm_gemm_f32(_p(x), _p(w), _p(out), M, N, Kd, self._stream()))
            else:
                self._check(self.lib.idm_gemm_bf16(_p(x), _p(w), _p(out), M, N, Kd, self._stream()))
        return out

    def gemm_choices(self, pair: Optional[bool] = None, lanes_up_to_tiles: Optional[int] = None,
                     band_mb: Optional[int] = None) -> None:
        """Which kernel a product of many tokens takes (tests compare them bit for bit; measurements): ``pair``:
        pairs of blocks on a tile where there are tiles enough, or never; ``lanes_up_to_tiles``: up to how many
        tiles of the persistent kernels a step of more than 128 tokens stays on the kernel with the tokens on the
        lanes; ``band_mb``: MB of the weight in a band of the persistent kernels' walk."""
        if self.dtype != torch.bfloat16:
            return
        if pair is not None:
            self.lib.idm_gemm_set_pair(1 if pair else 0, 0)
        if lanes_up_to_tiles is not None:
            self.lib.idm_gemm_set_small_tiles(int(lanes_up_to_tiles))
        if band_mb is not None:
            self.lib.idm_gemm_set_band_mb(int(band_mb))

    # ---- fused epilogues (bfloat16 only) ------------------------------------------------------------
    def gemm_residual(self, x, w, h) -> None:
        """``h += x . w^T`` in 32-bit, in place."""
        M, N, Kd = self._gemm_shape(x, w)
        self._need(h, torch.float32, "residual stream")
        if tuple(h.shape) != (M, N):
            raise KernelError(f"residual stream {tuple(h.shape)} does not match the product {(M, N)}")
        if M:
            self._check(self.lib.idm_gemm_bf16_residual(_p(x), _p(w), _p(h), M, N, Kd, self._stream()))

    def tile_gate_up(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        """Rows of gate and up alternating (gate row of a feature, then its up row), padded with zero
        rows to whole tiles of 64 features = 128 rows: the layout ``gemm_swiglu`` reads."""
        inter, Kd = gate.shape
        tiles = -(-inter // 64)
        out = torch.zeros((tiles * 64, 2, Kd), dtype=gate.dtype, device=gate.device)
        out[:inter, 0] = gate
        out[:inter, 1] = up
        return out.view(tiles * 128, Kd).contiguous()

    def gemm_swiglu(self, x, w_tiled, inter: int) -> torch.Tensor:
        """``silu(x . gate^T) * (x . up^T)`` in the storage dtype ``[M, inter]``."""
        M, N, Kd = self._gemm_shape(x, w_tiled)
        if N != -(-inter // 64) * 128:
            raise KernelError(f"tiled gate/up weight has {N} rows, expected {-(-inter // 64) * 128}")
        y = torch.empty((M, inter), dtype=self.dtype, device=self.device)
        if M:
            self._check(self.lib.idm_gemm_bf16_swiglu(_p(x), _p(w_tiled), _p(y), M, inter, Kd, self._stream()))
        return y

    QKV_FUSED_HEAD_DIMS = (32, 64, 128)

    def gemm_qkv(self, x, w, n_q, n_kv, hd, q_gamma, k_gamma, eps, cs, ctx, kv, keep_new: bool):
        """The fused q/k/v projection with norm, rotation and cache write as its epilogue
        (head_dim in ``QKV_FUSED_HEAD_DIMS``)."""
        M, N, Kd = self._gemm_shape(x, w)
        if N != (n_q + 2 * n_kv) * hd or hd not in self.QKV_FUSED_HEAD_DIMS:
            raise KernelError(f"gemm_qkv: weight rows {N}, heads {(n_q, n_kv)}, head_dim {hd}")
        if cs is not None and tuple(cs.shape) != (M, hd // 2, 2):
            raise KernelError(f"rotary table {tuple(cs.shape)} does not match {(M, hd // 2, 2)}")
        q = torch.empty((M, n_q, hd), dtype=self.dtype, device=self.device)
        k_new = v_new = None
        if keep_new and n_kv:
            k_new = torch.empty((M, n_kv, hd), dtype=self.dtype, device=self.device)
            v_new = torch.empty((M, n_kv, hd), dtype=self.dtype, device=self.device)
        if kv is not None:
            self._check_kv(kv, n_kv, hd)
        if M:
            self._check(self.lib.idm_gemm_bf16_qkv(
                _p(x), _p(w), M, Kd, n_q,
                n_kv, hd, _p(q_gamma), _p(k_gamma), eps,
                _p(cs), _p(getattr(cs, "by_dim", None)), _p(q), _p(k_new), _p(v_new),
                (_p(kv.k) if kv is not None else None), (_p(kv.v) if kv is not None else None),
                (_p(kv.table) if kv is not None else None),
                (kv.table.shape[1] if kv is not None else 0), (kv.ring if kv is not None else 0),
                _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), self._stream()))
        return q, k_new, v_new

    def wait_probe(self, limit_cycles: int, arrive: bool = False):
        """The kernels' bounded wait on a barrier nobody arrives at (or, with ``arrive``, one somebody does):
        returns (ran out, cycles waited, the second role left by the abort flag).  The kernel ends normally
        either way; a wait that ran out shows in ``gemm_status()``."""
        if self.dtype != torch.bfloat16:
            raise KernelError("the wait probe lives in the bfloat16 library")
        out = torch.full((3,), -1, dtype=torch.int32, device=self.device)
        self._check(self.lib.idm_wait_probe(int(limit_cycles), 1 if arrive else 0, _p(out), self._stream()), 1)
        ran_out, cycles, other = out.tolist()
        return bool(ran_out), int(cycles), bool(other)

    def gemm_status(self) -> int:
        """0, or 1 if a bounded wait inside the tensor-core GEMM ran out since the last call (synchronises)."""
        return 0 if self.dtype == torch.float32 else self.lib.idm_gemm_status()

    # ---- a norm without statistics, one-argument activations, streams side by side, capped logits ----
    def _delta_args(self, delta, n, hidden):
        if delta is None:
            return None, 0, 0
        self._need(delta, torch.float32, "delta")
        if delta.dim() != 3 or tuple(delta.shape[1:]) != (n, hidden):
            raise KernelError(f"delta {tuple(delta.shape)} does not match the stream {(n, hidden)}")
        return delta.data_ptr(), delta.shape[0], n * hidden

    def add_dyt(self, h, delta, w, b, alpha: float, rows=None) -> torch.Tensor:
        """``h += delta`` (in place, unless ``rows`` selects rows), then ``tanh(alpha h) * w + b`` in the storage dtype."""
        self._need(h, torch.float32, "residual stream")
        self._need(w, torch.float32, "norm weight")
        self._need(b, torch.float32, "norm bias")
        n, hidden = h.shape
        if w.numel() != hidden or b.numel() != hidden:
            raise KernelError(f"norm weight and bias have {w.numel()}, {b.numel()} elements, rows have {hidden}")
        dp, P, stride = self._delta_args(delta, n, hidden)
        if rows is not None:
            self._need(rows, torch.int32, "rows")
        n_out = n if rows is None else rows.numel()
        x = torch.empty((n_out, hidden), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_add_dyt(_p(h), dp, P, stride, _p(w), _p(b), float(alpha), _p(x), _p(rows), n_out, hidden,
                                         self._stream()))
        return x

    def act_cast(self, z: torch.Tensor, act: int) -> torch.Tensor:
        """An activation of one argument over a 32-bit product, in the storage dtype (``act`` 2: relu squared)."""
        self._need(z, torch.float32, "activation input")
        y = torch.empty(z.shape, dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_act_cast(_p(z), _p(y), z.numel(), act, self._stream()))
        return y

    def concat_cast(self, h, delta, x0) -> torch.Tensor:
        """``h += delta`` in place, then ``[h | x0]`` in the storage dtype ``[N, 2 * hidden]``."""
        self._need(h, torch.float32, "residual stream")
        self._need(x0, torch.float32, "second stream")
        n, hidden = h.shape
        if tuple(x0.shape) != (n, hidden):
            raise KernelError(f"streams {tuple(h.shape)} and {tuple(x0.shape)} differ")
        dp, P, stride = self._delta_args(delta, n, hidden)
        out = torch.empty((n, 2 * hidden), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_concat_cast(_p(h), dp, P, stride, _p(x0), _p(out), n, hidden, self._stream()))
        return out

    def logit_cap(self, logits: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
        """In place: ``cap * tanh(logits * scale / cap)`` (``cap`` 0: the constant alone)."""
        self._need(logits, torch.float32, "logits")
        self._check(self.lib.idm_logit_cap(_p(logits), logits.numel(), float(scale), float(cap or 0.0), self._stream()))
        return logits

    # ---- attention through a latent -----------------------------------------------------------------
    def latent_max_rank(self) -> int:
        return int(self.lib.idm_latent_attention_max_rank())

    def latent_kv_finish(self, proj, col0: int, rank: int, rot_dim: int, rot_dims: int, w_norm, eps: float, cs, mag: float,
                         kv, ctx, keep_rows: bool = False):
        """Columns ``[col0, col0 + rank + rot_dim)`` of the 32-bit ``proj``: the first ``rank`` normed (one root mean
        square, times ``w_norm``), the rest turned by the step's table ``cs [N, half, 2]``; the row goes to the
        token's place in the cache entry and, with ``keep_rows``, is also returned packed ``[N, rank + rot_dim]``."""
        self._need(proj, torch.float32, "projection")
        n, ld = proj.shape
        D = rank + rot_dim
        if kv.k.dtype != self.dtype or tuple(kv.k.shape[1:]) != (1, self.page, D) or not kv.k.is_contiguous():
            raise KernelError(f"cache entry {tuple(kv.k.shape)} {kv.k.dtype} does not fit [pages, 1, {self.page}, {D}]")
        half = 0 if cs is None else cs.shape[1]
        rows = torch.empty((n, D), dtype=self.dtype, device=self.device) if keep_rows else None
        self._check(self.lib.idm_latent_kv_finish(_p(proj), ld, col0, rank, rot_dim, rot_dims, _p(w_norm), eps, _p(cs), half,
                                                  float(mag), _p(kv.k), _p(kv.table), kv.table.shape[1], _p(ctx.token_seq),
                                                  _p(ctx.positions), _p(ctx.slots), _p(rows), n, self._stream()))
        return rows

    def headwise(self, x, x_col: int, n_heads: int, head_stride: int, w, tail: int = 0, rot_dims: int = 0, cs=None,
                 mag: float = 1.0, out_f32: bool = False) -> torch.Tensor:
        """A matrix per head: ``out[t, h, :O] = x[t, x_col + h * head_stride : ... + I] . w[h]`` with ``w [H, I, O]``;
        ``tail`` more columns of ``x`` behind a head's ``I`` are copied behind its outputs, the first ``rot_dims`` of them
        turned.  ``x`` 32-bit ``[N, ld]``; returns ``[N, H, O + tail]`` (32-bit or the storage dtype)."""
        self._need(x, torch.float32, "headwise input")
        self._need(w, self.dtype, "headwise matrices")
        n, ld = x.shape
        H, I, O = w.shape
        if H != n_heads or x_col + (H - 1) * head_stride + I + tail > ld:
            raise KernelError(f"headwise: {H} heads of {I}+{tail} columns, stride {head_stride}, from column {x_col} of {ld}")
        out = torch.empty((n, H, O + tail), dtype=torch.float32 if out_f32 else self.dtype, device=self.device)
        half = 0 if cs is None else cs.shape[1]
        self._check(self.lib.idm_headwise(x.data_ptr() + 4 * x_col, ld, head_stride, I, _p(w), O, _p(out), 1 if out_f32 else 0,
                                          H * (O + tail), O + tail, tail, rot_dims, _p(cs), half, float(mag), n, H,
                                          self._stream()))
        return out

    def latent_attention(self, qa, kv, ctx, rank: int, scale: float, sink=None) -> torch.Tensor:
        """Causal attention of the step's queries ``qa [N, H, D]`` (32-bit, in the latent's space) over the cached rows
        ``[c | r]`` of ``D`` numbers; returns the context ``[N, H * rank]`` in 32-bit: the weighted sums of ``c``.
        Steps of few tokens cut the keys into runs of 64 to 256 positions, a block each, that meet in scratch."""
        self._need(qa, torch.float32, "latent queries")
        n, H, D = qa.shape
        if tuple(kv.k.shape[1:]) != (1, self.page, D):
            raise KernelError(f"cache entry {tuple(kv.k.shape)} does not fit rows of {D}")
        if sink is not None:
            self._need(sink, torch.float32, "sink")
            if sink.numel() != H:
                raise KernelError(f"{sink.numel()} sinks for {H} heads")
        out = torch.empty((n, H * rank), dtype=torch.float32, device=self.device)
        run_keys, n_runs, part = 256, 1, None
        groups = n * (-(-H // self.lib.idm_latent_attention_heads_per_block(H, rank, D)))      # blocks per run
        if groups < 2 * self.sm_count:
            # runs short enough to give the step about four blocks per SM, of 64 to 256 keys (whole pages); the
            # choice depends on the step's shape and the cache's limit only, never on a sequence's length
            fair = -(-ctx.max_kv_len * groups // (4 * self.sm_count))
            run_keys = min(256, max(64, -(-fair // 64) * 64))
            run_keys = max(run_keys, -(-ctx.max_kv_len // (512 * 64)) * 64)       # (at most 512 runs)
            n_runs = max(1, -(-ctx.max_kv_len // run_keys))
        if n_runs > 1:
            part = self.scratch("latent_attention", n * H * n_runs * (rank + 2))
        else:
            run_keys = 1 << 30
        self._check(self.lib.idm_latent_attention(_p(qa), _p(kv.k), _p(kv.table), kv.table.shape[1], _p(ctx.token_seq),
                                                  _p(ctx.positions), _p(ctx.slots), _p(sink), _p(out), _p(part), n, H, rank,
                                                  D, scale, run_keys, n_runs, self._stream()), 2 if n_runs > 1 else 1)
        return out

    def latent_expand_pack(self, proj, up, rows, H, dn, dr, dv, R, rot_dims, cs, mag, hd, table, n_pages, ctx):
        """The operands of the per-head attention kernel for a step of whole prompts: ``q [N, H, hd]`` and pages of the
        step's own for k and v ``[n_pages, H, PAGE, hd]``, zero behind a head's own dims (see csrc/latent.cu)."""
        n = proj.shape[0]
        q = torch.empty((n, H, hd), dtype=self.dtype, device=self.device)
        k = torch.empty((n_pages, H, self.page, hd), dtype=self.dtype, device=self.device)
        v = torch.empty((n_pages, H, self.page, hd), dtype=self.dtype, device=self.device)
        half = 0 if cs is None else cs.shape[1]
        self._check(self.lib.idm_latent_expand_pack(_p(proj), proj.shape[1], _p(up), _p(rows), H, dn, dr, dv, R, rot_dims, _p(cs),
                                                    half, float(mag), hd, _p(q), _p(k), _p(v), _p(table), table.shape[1],
                                                    _p(ctx.token_seq), _p(ctx.positions), _p(ctx.slots), n, self._stream()))
        return q, k, v

    # ---- experts chosen per token -------------------------------------------------------------------
    # from this many (token, choice) pairs on, a step of few tokens walks its experts one by one
    EXPERT_MAJOR_FROM = 64

    def experts_few(self, x, tokens, table, gate_up, row_stride: int, up_off: int, down, h, act: int, weight: float,
                    pair_w=None) -> None:
        """``h[t] += weight * sum_k down[e] (act(gate[e] x_t) * up[e] x_t)``, ``e = table[tokens[t], k]``: every (token, choice)
        streams its expert's matrices (steps of few tokens).  ``gate_up [E, rows, width]`` holds an expert's gate and up
        rows: gate row f starts ``f * row_stride`` elements into the expert's block and its up row ``up_off`` behind it.
        ``down [E, width, ff]``."""
        self._need(x, self.dtype, "experts input")
        self._need(h, torch.float32, "residual stream")
        self._need(gate_up, self.dtype, "experts' gate and up rows")
        self._need(down, self.dtype, "experts' down matrices")
        self._need(tokens, torch.int32, "tokens")
        self._need(table, torch.int32, "expert table")
        n, width = x.shape
        E, _, ff = down.shape
        top = table.shape[1]
        if gate_up.shape[0] != E or gate_up.shape[2] != width or (ff - 1) * row_stride + up_off + width > gate_up.shape[1] * width:
            raise KernelError(f"experts: gate/up rows {tuple(gate_up.shape)} do not hold {ff} rows at stride {row_stride} + {up_off}")
        a = torch.empty((n, top, ff), dtype=torch.float32, device=self.device)
        if n * top > self.EXPERT_MAJOR_FROM and max(width, ff) * 32 + n * top * 4 <= 200 * 1024:
            # more pairs than a few: expert by expert, so that an expert's matrices are read once a step
            # (zeros: a pair that names no expert of these has no block, and its row is added as it lies)
            z = torch.zeros((n * top, width), dtype=torch.float32, device=self.device)
            self._check(self.lib.idm_experts_major(_p(x), _p(tokens), _p(table), _p(pair_w), _p(gate_up), gate_up.shape[1] * width, row_stride,
                                                   up_off, _p(down), _p(a), _p(z), _p(h), n, width, ff, top, E, act, float(weight),
                                                   self._stream()), 3)
            return
        self._check(self.lib.idm_experts_few(_p(x), _p(tokens), _p(table), _p(pair_w), _p(gate_up), gate_up.shape[1] * width, row_stride, up_off, _p(down),
                                             _p(a), _p(h), n, width, ff, top, E, act, float(weight), self._stream()), 2)

    def rows_gather(self, x, src) -> torch.Tensor:
        self._need(x, self.dtype, "rows")
        self._need(src, torch.int32, "row numbers")
        out = torch.empty((src.numel(), x.shape[1]), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_rows_gather(_p(x), _p(src), _p(out), src.numel(), x.shape[1], self._stream()))
        return out

    def experts_dense(self, x, tokens, table, gate_up, down, h, act: int, weight: float, pair_w=None) -> None:
        """``h[t] += weight * sum_k ff_e(x_t)``, ``e = table[tokens[t], k]``, by running EVERY expert over all the step's
        tokens with the library's matrix products and letting each token pick its own (single-token steps of many
        sequences: every expert's matrices are streamed once, in shapes that do not change from step to step)."""
        self._need(x, self.dtype, "experts input")
        self._need(h, torch.float32, "residual stream")
        n, width = x.shape
        E, _, ff = down.shape
        y = torch.empty((n, ff), dtype=self.dtype, device=self.device)
        z = torch.empty((E, n, width), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_experts_dense(_p(x), _p(tokens), _p(table), _p(pair_w), E, _p(gate_up), gate_up.shape[1] * width, _p(down),
                                               width * ff, _p(y), _p(z), _p(h), n, width, ff, table.shape[1], act, float(weight),
                                               self._stream()), 2 * E + 1)

    def experts_grouped_step(self, x, src, place, counts, gate_up, down, h, act: int, weight: float, pair_w=None) -> None:
        """A step's rows grouped by expert through every expert's gated feed-forward, from one call into the library:
        rows gathered in the order of their experts (``src [rows]``: grouped row -> token), the gated product (activation
        in its epilogue, ``gate_up`` in the layout of ``tile_gate_up``) and the down product of every expert that has
        rows (``counts``: rows per expert, a contiguous int32 numpy array on the host), and the outputs added into ``h``
        in the order of a token's choices (``place [tokens, top]``: (token, choice) -> grouped row)."""
        self._need(x, self.dtype, "experts input")
        self._need(h, torch.float32, "residual stream")
        n, width = x.shape
        E, _, ff = down.shape
        top = place.shape[1]
        xg = torch.empty((n * top, width), dtype=self.dtype, device=self.device)
        y = torch.empty((n * top, ff), dtype=self.dtype, device=self.device)
        z = torch.empty((n * top, width), dtype=torch.float32, device=self.device)
        with_rows = int((counts > 0).sum())
        self._check(self.lib.idm_experts_grouped_step(_p(x), _p(src), _p(place), _p(pair_w), counts.ctypes.data, E, _p(gate_up),
                                                      gate_up.shape[1] * width, _p(down), width * ff, _p(xg), _p(y), _p(z), _p(h),
                                                      n, top, width, ff, act, float(weight), self._stream()), 2 * with_rows + 2)

    def dense_ff(self, x, w_up, w_down, h, act: int) -> None:
        """``h += w_down . act(w_up . x)`` from one call: the up product, the activation, the down product with the sum
        into the stream as its epilogue (bfloat16)."""
        M, ff, Kd = self._gemm_shape(x, w_up)
        self._need(w_down, self.dtype, "down weight")
        self._need(h, torch.float32, "residual stream")
        if tuple(w_down.shape) != (Kd, ff) or tuple(h.shape) != (M, Kd) or ff % 8:
            raise KernelError(f"dense_ff: up {tuple(w_up.shape)}, down {tuple(w_down.shape)}, stream {tuple(h.shape)}")
        z = torch.empty((M, ff), dtype=torch.float32, device=self.device)
        y = torch.empty((M, ff), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_dense_ff(_p(x), _p(w_up), _p(w_down), _p(z), _p(y), _p(h), M, Kd, ff, act, self._stream()), 3)

    def experts_combine(self, z, place, h, weight: float, pair_w=None) -> None:
        """``h[t] += weight * sum_k pair_w[t, k] * z[place[t, k]]`` in ascending k (``place`` < 0: nothing; no ``pair_w``: 1)."""
        self._need(z, torch.float32, "experts output")
        self._need(place, torch.int32, "places")
        n, width = h.shape
        self._check(self.lib.idm_experts_combine(_p(z), _p(place), _p(pair_w), _p(h), n, width, place.shape[1], float(weight), self._stream()))

    def route(self, z, correction, top: int, groups: int, keep: int, scale: float):
        """From 32-bit router logits ``z [N, E]`` to the experts each token uses: softmax over all E, choice by
        ``softmax + correction`` among the experts of the ``keep`` best of ``groups`` equal groups of neighbours, the
        ``top`` best in descending order; returns ``(chosen [N, top] int32, weight [N, top])`` with the weights the
        chosen experts' softmax values over their sum, times ``scale``."""
        self._need(z, torch.float32, "router logits")
        n, E = z.shape
        if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
            raise KernelError(f"route: the correction must hold one 32-bit number for each of the {E} experts")
        chosen = torch.empty((n, top), dtype=torch.int32, device=self.device)
        weight = torch.empty((n, top), dtype=torch.float32, device=self.device)
        self._check(self.lib.idm_route(_p(z), z.stride(0), _p(correction), _p(chosen), _p(weight), n, E, int(top), int(groups),
                                       int(keep), float(scale), self._stream()))
        return chosen, weight

    def experts_identity(self, x, chosen, weight, h, n_real: int) -> None:
        """``h[t] += x[t] * (the weights of t's pairs whose expert number is at least n_real)``: experts that hand
        their input on."""
        self._need(x, self.dtype, "experts input")
        self._need(h, torch.float32, "residual stream")
        n, width = x.shape
        self._check(self.lib.idm_experts_identity(_p(x), _p(chosen), _p(weight), _p(h), n, width, chosen.shape[1], int(n_real),
                                                  self._stream()))

    def post_layernorm(self, h, y, w, b, scale, eps: float, cast: bool = False):
        """``h += scale * layernorm(y)`` in place (``scale`` [hidden] or None); returns ``h`` in the storage dtype if
        ``cast`` (what a sublayer without a norm in front of it reads), else None."""
        self._need(h, torch.float32, "residual stream")
        self._need(y, torch.float32, "sublayer output")
        n, hidden = h.shape
        if tuple(y.shape) != (n, hidden) or w.numel() != hidden or b.numel() != hidden or (scale is not None and scale.numel() != hidden):
            raise KernelError(f"post_layernorm: stream {tuple(h.shape)}, output {tuple(y.shape)}, weight {w.numel()}")
        x = torch.empty((n, hidden), dtype=self.dtype, device=self.device) if cast else None
        self._check(self.lib.idm_post_layernorm(_p(h), _p(y), _p(w), _p(b), _p(scale), float(eps), _p(x), 2 if cast else 0, n,
                                                hidden, self._stream()))
        return x

    def add_layernorm(self, h, delta, w, b, eps: float, rows=None) -> torch.Tensor:
        """``h += delta`` in place (unless ``rows`` picks rows), then ``layernorm(h) * w + b`` in the storage dtype."""
        self._need(h, torch.float32, "residual stream")
        n, hidden = h.shape
        dp, P, stride = self._delta_args(delta, n, hidden)
        if rows is not None:
            self._need(rows, torch.int32, "rows")
        n_out = n if rows is None else rows.numel()
        x = torch.empty((n_out, hidden), dtype=self.dtype, device=self.device)
        self._check(self.lib.idm_add_layernorm(_p(h), dp, P, stride, _p(w), _p(b), float(eps), _p(x), _p(rows), n_out,
                                               hidden, self._stream()))
        return x

    def embed_bigram(self, ctx, table, bigram, last, buckets: int, mul_prev: int, mul_cur: int, cast: bool = False):
        """The 32-bit stream ``table[token] + bigram[row]`` with ``row = (previous token * mul_prev + token * mul_cur) %
        buckets``, the table's last row for a sequence's first token; ``last [slots, 1]`` int32 holds every sequence's
        last token between steps and is moved on.  Returns ``(h, h in the storage dtype or None)``."""
        self._need(table, self.dtype, "embed table")
        self._need(bigram, self.dtype, "bigram table")
        if last.dtype != torch.int32 or last.dim() != 2 or bigram.shape[0] != buckets + 1 or bigram.shape[1] != table.shape[1]:
            raise KernelError(f"embed_bigram: table {tuple(bigram.shape)} for {buckets} buckets, state {tuple(last.shape)} {last.dtype}")
        n, hidden = ctx.tokens.numel(), table.shape[1]
        h = torch.empty((n, hidden), dtype=torch.float32, device=self.device)
        x = torch.empty((n, hidden), dtype=self.dtype, device=self.device) if cast else None
        self._check(self.lib.idm_embed_bigram(_p(ctx.tokens), _p(ctx.token_seq), _p(ctx.positions), _p(ctx.cu_q), _p(ctx.slots),
                                              _p(table), _p(bigram), _p(last), last.stride(0), _p(h), _p(x), n, hidden,
                                              int(buckets), int(mul_prev), int(mul_cur), self._stream()))
        return h, x

    def sample(self, logits: torch.Tensor, temperature: float, keys: Optional[torch.Tensor]) -> torch.Tensor:
        self._need(logits, torch.float32, "logits")
        B, V = logits.shape
        if keys is not None:
            self._need(keys, torch.int64, "row keys")
            if keys.numel() != B:
                raise KernelError("one key per row")
        out = torch.empty((B,), dtype=torch.int32, device=self.device)
        scratch = self.scratch("sample", self.lib.idm_sample_scratch_floats(B, V))
        self._check(self.lib.idm_sample(_p(logits), B, V, temperature,
                                        _p(keys), _p(out), _p(scratch), self._stream()))
        return out


    def decode_advance(self, tokens, positions, q_start, kv_len, sampled, history, step_counter) -> None:
        """tokens <- sampled; positions, q_start, kv_len += 1; history[step] <- sampled; step += 1."""
        n = tokens.numel()
        self._check(self.lib.idm_decode_advance(
            _p(tokens), _p(positions), _p(q_start), _p(kv_len),
            _p(sampled), _p(history), _p(step_counter), n,
            history.shape[0], self._stream()))
