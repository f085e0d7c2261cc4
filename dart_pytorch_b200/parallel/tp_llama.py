"""Tensor-parallel Llama inference engine: batched prefill and greedy decode with a device-resident KV cache.

The reference runs Llama one sequence at a time on one device (lib/core/nn/llama.dart:186-330) and has no tensor
parallelism.  Here every rank of a tensor-parallel group holds ``1/T`` of the query / KV heads and of the feed-forward
width.  Per block and rank:

    y   = rmsnorm(x)                                  (replicated)
    qkv = y @ Wqkv_r^T                                column-parallel, no communication
    rope(q, k); K / V rows appended to this rank's cache (one fused kernel)
    o   = attention(q, cache)                         flash kernel for prefill, split-KV decode kernel for few rows
    x'  = x + sum_r(o_r @ Wo_r^T)                     row-parallel: ONE kernel, GEMM + all-reduce over NVLink
    y   = rmsnorm(x');  h = silu(y Wg_r^T) * (y Wu_r^T)
    x   = x' + sum_r(h_r @ Wd_r^T)                    row-parallel: ONE kernel again

The residual stream ping-pongs between two symmetric activation buffers.  Prefill also has a sequence-parallel schedule
(``prefill(..., mode="sp")``): the residual stream is sharded by rows, every rank normalises only its rows, the
column-parallel GEMMs read the peers' normalised rows in place (all-gather fused into the GEMM's operand loads) and the
row-parallel GEMMs end in a reduce-scatter instead of an all-reduce, which halves the NVLink bytes per projection pair
and divides the norm work by the group size.  The output head is vocabulary-sharded; the
greedy token is picked by one kernel that exchanges per-rank (max, index) pairs through peer memory, so a decode step
never returns to the host and is captured in a CUDA graph (the position lives in device memory).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..models.llama import Llama, LlamaConfig
from ..ops import decode as D
from ..ops import flash
from ..ops import kernels as K
from ..utils import trace
from .tp import MAX_RANKS, TpComm, shard_range

c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


class TpArgmaxArgs(ctypes.Structure):
    _fields_ = [("logits", c_void_p), ("ld", c_ll), ("B", c_int), ("Vl", c_int), ("vocab_offset", c_int),
                ("rank", c_int), ("world", c_int), ("xchg_peer", c_void_p * MAX_RANKS),
                ("flags_peer", c_void_p * MAX_RANKS), ("tokens", c_void_p), ("epoch", c_void_p),
                ("exit_counter", c_void_p), ("pos_ptr", c_void_p), ("pos_inc", c_int)]


class _Layer:
    __slots__ = ("attn_norm", "w_qkv", "wo", "ffn_norm", "w_gate_up", "w_down", "k_cache", "v_cache")


class TPLlamaEngine:
    def __init__(self, config: LlamaConfig, max_batch: int, max_ctx: int, max_rows: int, group=None, seed: int = 0,
                 init_std: float = 0.02, full_model: Optional[Llama] = None, use_nvls: Optional[bool] = None):
        """``max_rows``: the largest number of token rows one forward call processes (prefill chunk or decode batch).
        Weights are random N(0, init_std) shards unless ``full_model`` (a whole ``Llama`` present on every rank) is
        given, in which case this rank's shards are sliced out of it."""
        import torch.distributed._symmetric_memory as symm_mem
        c = config
        self.config = c
        self.group = group if group is not None else dist.group.WORLD
        self.T, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        T, r = self.T, self.rank
        if c.num_heads % T or c.num_kv_heads % T or c.ffn_dim % T or c.vocab_size % T:
            raise ValueError("TPLlamaEngine: heads, kv heads, ffn width and vocabulary must divide by the group size")
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.hd = c.head_dim
        self.Hq, self.Hkv, self.F, self.Vl = c.num_heads // T, c.num_kv_heads // T, c.ffn_dim // T, c.vocab_size // T
        self.max_batch, self.max_ctx, self.max_rows = max_batch, max_ctx, max_rows
        # three activation buffers: the sequence-parallel prefill keeps x, norm(x) and x' apart
        self.comm = TpComm(max_rows, c.embed_dim, group=self.group, num_bufs=3, use_nvls=use_nvls)
        self.lib = N.load()
        self.lib.dptb_tp_argmax.argtypes = [ctypes.POINTER(TpArgmaxArgs), c_void_p]
        self.lib.dptb_tp_argmax.restype = c_int
        bf = dict(device=self.dev, dtype=torch.bfloat16)
        d, hd = c.embed_dim, self.hd
        gen = torch.Generator(device=self.dev).manual_seed(seed * 1000 + r)
        shared = torch.Generator(device=self.dev).manual_seed(seed * 1000 + 999)   # replicated tensors: same on all ranks

        def rnd(rows, cols, g=gen):
            return (torch.randn(rows, cols, device=self.dev, generator=g) * init_std).to(torch.bfloat16)
        q0, q1 = shard_range(c.num_heads, r, T)
        k0, k1 = shard_range(c.num_kv_heads, r, T)
        f0, f1 = shard_range(c.ffn_dim, r, T)
        v0, v1 = shard_range(c.vocab_size, r, T)
        self.vocab_offset = v0
        if full_model is None:
            self.embed = rnd(c.vocab_size, d, shared)
            self.final_norm = torch.ones(d, **bf)
            self.head = self.embed[v0:v1] if c.tie_weights else rnd(self.Vl, d)
        else:
            m = full_model
            self.embed = m.embed_in.weight.detach().to(**bf).contiguous()
            self.final_norm = m.final_norm.gamma.detach().to(**bf).contiguous()
            self.head = m.head_weight.detach().to(**bf)[v0:v1].contiguous()
        self.layers: List[_Layer] = []
        for li in range(c.num_layers):
            L = _Layer()
            if full_model is None:
                L.attn_norm, L.ffn_norm = torch.ones(d, **bf), torch.ones(d, **bf)
                L.w_qkv = rnd((self.Hq + 2 * self.Hkv) * hd, d)
                L.wo = rnd(d, self.Hq * hd)
                L.w_gate_up = rnd(2 * self.F, d)
                L.w_down = rnd(d, self.F)
            else:
                blk = full_model.blocks[li]
                W = blk.attn.w_qkv.detach().to(**bf)
                H, Hk = c.num_heads, c.num_kv_heads
                L.w_qkv = torch.cat([W[q0 * hd:q1 * hd], W[(H + k0) * hd:(H + k1) * hd],
                                     W[(H + Hk + k0) * hd:(H + Hk + k1) * hd]], 0).contiguous()
                L.wo = blk.attn.wo.weight.detach().to(**bf)[:, q0 * hd:q1 * hd].contiguous()
                L.attn_norm = blk.attn_norm.gamma.detach().to(**bf).contiguous()
                L.ffn_norm = blk.ffn_norm.gamma.detach().to(**bf).contiguous()
                gu = blk.ffn.w_gate_up.detach().to(**bf)              # [gate rows | up rows]
                Fh = c.ffn_dim
                L.w_gate_up = torch.cat([gu[f0:f1], gu[Fh + f0:Fh + f1]], 0).contiguous()
                L.w_down = blk.ffn.down.weight.detach().to(**bf)[:, f0:f1].contiguous()
            L.k_cache = torch.zeros(max_batch, max_ctx, self.Hkv * hd, **bf)
            L.v_cache = torch.zeros(max_batch, max_ctx, self.Hkv * hd, **bf)
            self.layers.append(L)
        # decode scratch (fixed addresses: the decode step is captured in a CUDA graph)
        ws = D.decode_workspace_floats(max_batch, 1, self.Hq, self.Hkv, hd, max_ctx)
        self.dec_ws = torch.empty(max(ws, 1), dtype=torch.float32, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.tokens = torch.zeros(max_batch, dtype=torch.long, device=self.dev)
        self.logits = torch.empty(max_batch, self.Vl, **bf)
        gname = self.group.group_name
        self._xchg = symm_mem.empty(2 * max_batch * MAX_RANKS * 2, dtype=torch.float32, device=self.dev)
        self._xchg.zero_()
        self._h_xchg = symm_mem.rendezvous(self._xchg, group=gname)
        self._aflags = symm_mem.empty(max_batch * MAX_RANKS, dtype=torch.int32, device=self.dev)
        self._aflags.zero_()
        self._h_aflags = symm_mem.rendezvous(self._aflags, group=gname)
        self._aepoch = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self._aexit = torch.zeros(1, dtype=torch.int32, device=self.dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._graph = None
        self._graph_batch = 0
        self.seq_len = 0

    # ---- pieces -----------------------------------------------------------------------------------------
    def _argmax(self, logits: torch.Tensor, B: int, advance: int) -> None:
        a = TpArgmaxArgs()
        a.logits, a.ld, a.B, a.Vl, a.vocab_offset = logits.data_ptr(), logits.stride(0), B, self.Vl, self.vocab_offset
        a.rank, a.world = self.rank, self.T
        for r in range(MAX_RANKS):
            a.xchg_peer[r] = int(self._h_xchg.buffer_ptrs[r]) if r < self.T else None
            a.flags_peer[r] = int(self._h_aflags.buffer_ptrs[r]) if r < self.T else None
        a.tokens, a.epoch, a.exit_counter = self.tokens.data_ptr(), self._aepoch.data_ptr(), self._aexit.data_ptr()
        a.pos_ptr, a.pos_inc = (self.pos.data_ptr(), advance) if advance else (None, 0)
        N.check(self.lib.dptb_tp_argmax(ctypes.byref(a), N.stream_ptr()), "tp_argmax")

    def _blocks(self, x: torch.Tensor, B: int, S: int, pos0: int, device_pos: bool) -> torch.Tensor:
        """Run all blocks on ``x`` = activation buffer 0 rows ``[B*S, D]``; returns the final residual stream (buffer 0)."""
        c, hd, Hq, Hkv = self.config, self.hd, self.Hq, self.Hkv
        M = B * S
        dq = Hq * hd
        pos = self.pos if device_pos else None
        decode_like = S <= 4
        for L in self.layers:
            y, _ = K.rmsnorm_fwd(x, L.attn_norm, c.rms_norm_eps)
            qkv = torch.empty(M, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device=self.dev)
            K.gemm(y, L.w_qkv, qkv, trans_b=True)
            D.rope_kv_append(qkv, L.k_cache, L.v_cache, B, S, Hq, Hkv, hd, pos0, base=c.rope_base, pos=pos)
            if decode_like:
                o = D.attn_decode(qkv[:, :dq], L.k_cache, L.v_cache, B, S, self.max_ctx if device_pos else pos0 + S,
                                  Hq, Hkv, hd, pos0, workspace=self.dec_ws, pos=pos)
            else:
                kf = L.k_cache.view(-1, Hkv * hd)
                vf = L.v_cache.view(-1, Hkv * hd)
                o, _ = flash.attn_fwd(qkv[:, :dq], kf, vf, B, S, pos0 + S, Hq, Hkv, hd, True, q_offset=pos0,
                                      need_lse=False, kv_batch_rows=self.max_ctx)
            x1 = self.comm.gemm_allreduce(o, L.wo, 1, residual=x)
            y2, _ = K.rmsnorm_fwd(x1, L.ffn_norm, c.rms_norm_eps)
            gu = torch.empty(M, 2 * self.F, dtype=torch.bfloat16, device=self.dev)
            K.gemm(y2, L.w_gate_up, gu, trans_b=True)
            h = K.swiglu_fwd(gu[:, :self.F], gu[:, self.F:])
            x = self.comm.gemm_allreduce(h, L.w_down, 0, residual=x1)
        return x

    def _blocks_sp(self, x: torch.Tensor, B: int, S: int) -> torch.Tensor:
        """Sequence-parallel schedule of ``_blocks`` for a prefill from position 0.  ``x``: this rank's rows
        ``[rank * M / T, (rank + 1) * M / T)`` of the embedded tokens, in activation buffer 0 (first ``M / T`` rows);
        returns this rank's rows of the final residual stream (same place).  Buffer 1 holds the normalised rows the
        peers read, buffer 2 the post-attention residual.  A buffer is rewritten only after a reduce-scatter GEMM has
        completed in between: that kernel ends with a handshake of all ranks, so every rank's earlier reads are over."""
        c, hd, Hq, Hkv = self.config, self.hd, self.Hq, self.Hkv
        M = B * S
        Ms = M // self.T
        dq = Hq * hd
        for L in self.layers:
            y = self.comm.buffer(1, Ms)
            K.rmsnorm_fwd(x, L.attn_norm, c.rms_norm_eps, out=y)
            self.comm.publish_shard()
            qkv = torch.empty(M, (Hq + 2 * Hkv) * hd, dtype=torch.bfloat16, device=self.dev)
            self.comm.allgather_gemm(1, Ms, L.w_qkv, qkv)
            D.rope_kv_append(qkv, L.k_cache, L.v_cache, B, S, Hq, Hkv, hd, 0, base=c.rope_base, pos=None)
            kf = L.k_cache.view(-1, Hkv * hd)
            vf = L.v_cache.view(-1, Hkv * hd)
            o, _ = flash.attn_fwd(qkv[:, :dq], kf, vf, B, S, S, Hq, Hkv, hd, True, q_offset=0, need_lse=False,
                                  kv_batch_rows=self.max_ctx)
            x1 = self.comm.gemm_reduce_scatter(o, L.wo, 2, residual=x)
            y2 = self.comm.buffer(1, Ms)
            K.rmsnorm_fwd(x1, L.ffn_norm, c.rms_norm_eps, out=y2)
            self.comm.publish_shard()
            gu = torch.empty(M, 2 * self.F, dtype=torch.bfloat16, device=self.dev)
            self.comm.allgather_gemm(1, Ms, L.w_gate_up, gu)
            h = K.swiglu_fwd(gu[:, :self.F], gu[:, self.F:])
            x = self.comm.gemm_reduce_scatter(h, L.w_down, 0, residual=x1)
        return x

    def _gather_last_rows(self, nb: int, S: int) -> torch.Tensor:
        """Last-token rows ``[nb, D]`` of a row-sharded residual stream in buffer 0: each row is fetched from the rank
        that owns it with this package's gather kernel reading the peer's buffer in place (plain loads over NVLink)."""
        M = nb * S
        Ms = M // self.T
        out = torch.empty(nb, self.config.embed_dim, dtype=torch.bfloat16, device=self.dev)
        rows = torch.arange(nb, device=self.dev) * S + (S - 1)
        h = self.comm._h_bufs[0]
        for r in range(self.T):
            sel = ((rows >= r * Ms) & (rows < (r + 1) * Ms)).nonzero().view(-1)
            if sel.numel() == 0:
                continue
            src = self.comm.bufs[0] if r == self.rank else \
                h.get_buffer(r, (self.comm.max_rows, self.comm.width), torch.bfloat16)
            out[sel] = K.embedding_fwd(src[:Ms], (rows[sel] - r * Ms))
        return out

    def _head(self, x_last: torch.Tensor, B: int, advance: int) -> None:
        xf, _ = K.rmsnorm_fwd(x_last, self.final_norm, self.config.rms_norm_eps)
        K.gemm(xf, self.head, self.logits[:B], trans_b=True)
        self._argmax(self.logits[:B], B, advance)

    # ---- public API -------------------------------------------------------------------------------------
    def reset(self) -> None:
        self.seq_len = 0
        self.pos.zero_()

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, chunk: Optional[int] = None, mode: str = "ar") -> torch.Tensor:
        """``tokens [B, S]`` (the same on every rank).  Fills the caches and returns the first generated token ids
        ``[B]`` (device).  Sequences are processed ``chunk`` at a time so the rows of a call fit ``max_rows``.
        ``mode``: "ar" keeps activations replicated (GEMM + all-reduce); "sp" shards them by rows (GEMM +
        reduce-scatter, all-gather + GEMM) and needs the rows of a call to split into whole 128-row tiles per rank
        (it falls back to "ar" for chunks that do not)."""
        if mode not in ("ar", "sp"):
            raise ValueError("prefill: mode must be 'ar' or 'sp'")
        B, S = tokens.shape
        if B > self.max_batch or S > self.max_ctx:
            raise ValueError("prefill: batch or sequence exceeds the engine's capacity")
        if self.seq_len != 0:
            raise ValueError("prefill: call reset() first")
        chunk = chunk or max(1, self.max_rows // S)
        if chunk * S > self.max_rows:
            raise ValueError(f"prefill: {chunk} sequences of {S} tokens exceed max_rows={self.max_rows}")
        tokens = tokens.to(self.dev)
        last = torch.empty(B, self.config.embed_dim, dtype=torch.bfloat16, device=self.dev)
        for b0 in range(0, B, chunk):
            b1 = min(B, b0 + chunk)
            nb = b1 - b0
            sp = mode == "sp" and self.T > 1 and (nb * S) % (self.T * 128) == 0
            if sp:
                Ms = nb * S // self.T
                x = self.comm.buffer(0, Ms)
                x.copy_(K.embedding_fwd(self.embed, tokens[b0:b1].reshape(-1)[self.rank * Ms:(self.rank + 1) * Ms]))
            else:
                x = self.comm.buffer(0, nb * S)
                x.copy_(K.embedding_fwd(self.embed, tokens[b0:b1].reshape(-1)))
            views = []
            for L in self.layers:      # the chunk's sequences address their own cache rows
                views.append((L.k_cache, L.v_cache))
                L.k_cache, L.v_cache = L.k_cache[b0:b1], L.v_cache[b0:b1]
            try:
                with trace.range("tp/prefill_chunk"):
                    xo = self._blocks_sp(x, nb, S) if sp else self._blocks(x, nb, S, 0, device_pos=False)
            finally:
                for L, (kc, vc) in zip(self.layers, views):
                    L.k_cache, L.v_cache = kc, vc
            if sp:
                last[b0:b1] = self._gather_last_rows(nb, S)
                dist.barrier(group=self.group)     # peers have fetched their rows before buffer 0 is reused
            else:
                last[b0:b1] = xo.view(nb, S, -1)[:, -1, :]
        self.seq_len = S
        self.pos.fill_(S)
        self._head(last, B, advance=0)
        return self.tokens[:B].clone()

    def _decode_body(self, B: int) -> None:
        # The weight-streaming GEMMs of the step are launched as programmatic dependents of the small kernel before
        # them (norm, attention, SwiGLU): their set-up and first ring-full of weight tiles overlap that kernel.
        pdl = os.environ.get("DPTB200_TP_PDL", "1") != "0"
        lib = N.load()
        lib.dptb_gemm_skinny_set_pdl(1 if pdl else 0)
        try:
            with trace.range("tp/decode_step"):
                x = self.comm.buffer(0, B)
                x.copy_(K.embedding_fwd(self.embed, self.tokens[:B]))
                xo = self._blocks(x, B, 1, 0, device_pos=True)
                self._head(xo, B, advance=1)
        finally:
            lib.dptb_gemm_skinny_set_pdl(0)

    @torch.no_grad()
    def decode_step(self, B: int, use_graph: bool = True) -> torch.Tensor:
        """One greedy token for every sequence: consumes ``self.tokens`` (the previous step's output), appends to the
        caches at the device-resident position and leaves the new ids in ``self.tokens``."""
        if self.seq_len + 1 > self.max_ctx:
            raise ValueError("decode_step: the KV cache is full")
        if use_graph:
            if self._graph is None or self._graph_batch != B:
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                saved = (self.pos.clone(), self.tokens.clone())
                with torch.cuda.stream(s):
                    self._decode_body(B)                      # warm-up on the capture stream (allocations, tuning)
                    torch.cuda.synchronize()
                    dist.barrier(group=self.group)
                    self.pos.copy_(saved[0])
                    self.tokens.copy_(saved[1])
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=s):
                        self._decode_body(B)
                torch.cuda.current_stream().wait_stream(s)
                self._graph, self._graph_batch = g, B
                self.pos.copy_(saved[0])
                self.tokens.copy_(saved[1])
            self._graph.replay()
        else:
            self._decode_body(B)
        self.seq_len += 1
        return self.tokens[:B]

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy continuation of equal-length prompts ``[B, S]``; returns ``[B, S + max_new_tokens]`` ids."""
        self.reset()
        B = prompts.shape[0]
        out = [prompts.to(self.dev), self.prefill(prompts).view(B, 1)]
        for _ in range(max_new_tokens - 1):
            out.append(self.decode_step(B, use_graph).clone().view(B, 1))
        return torch.cat(out, dim=1)
