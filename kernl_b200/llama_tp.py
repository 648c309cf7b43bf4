"""Llama-2-shaped decoder on the kernl_b200 ops, with Megatron-style tensor parallelism.

This is the host side of the baseline's fifth config (32 layers, hidden 4096, 32 heads of 128,
SwiGLU 11008, RMSNorm eps 1e-5, rotary base 10000, vocab 32000, bf16): prefill with a causal mask,
then greedy decode with a KV cache. The reference has no such model in its dispatched path; the
semantics of the pieces follow its experimental Llama kernels
(experimental/llama-v2/kernel/pytorch_reference.py:6-8,37-80,88-104: RMSNorm, interleaved-pair
rotary embedding, silu(gate)·up), and every heavy op is one of the library's kernels:
RMSNorm (kb_norm_fwd), QKV / O / down projections and the gate-up projection with its silu·mul
epilogue (kb_linear_fwd), causal prefill attention (kb_attention_fwd), decode attention (kb_attention_decode_fwd).

Partitioning over `world` ranks (one process per GPU): heads are split (q/k/v column-parallel, the
KV cache is sharded by head, attention is local), `o_proj` and `down_proj` are row-parallel and
followed by an all-reduce (sum) over NVLink through `torch.distributed` (NCCL), gate/up are
column-parallel. Embedding and LM head are replicated.

Decode is shape-static so that ONE CUDA graph serves every step: the position / cache slot and the
number of filled slots are device tensors that the rotary and the decode-attention kernels read
(the `start_position` of experimental/llama-v2/kernel/fused_kernel_attention.py:30,63,76), so a
step streams only the keys that exist. Ops without that feature (the CPU stand-ins of the tests)
get an additive length mask instead.
"""
import os
from dataclasses import dataclass
from typing import Optional

import torch

from kernl_b200.comm import NcclAllReduce
from kernl_b200.implementations.linear_layer import interleave_gate_up


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    eps: float = 1e-5
    rope_base: float = 10000.0
    max_seq: int = 2304  # prefill 2048 + 256 decoded tokens


class CudaOps:
    """The library's kernels behind the five ops the model needs."""

    needs_len_mask = False  # decode attention reads the number of filled cache slots from the device

    @staticmethod
    def rms_norm(x, w, eps):
        from kernl_b200.implementations.layer_norm import layer_norm

        return layer_norm(x, w, None, eps, use_rms_norm=True)

    @staticmethod
    def linear(x, w, out=None):
        from kernl_b200.implementations.linear_layer import linear_layer

        return linear_layer(x, w, None, out=out)

    @staticmethod
    def gated_linear(x, w_gate_up):
        """silu(x · w_gateᵀ) * (x · w_upᵀ) in one GEMM whose epilogue does the gating; rows of
        `w_gate_up` as `interleave_gate_up` lays them out."""
        from kernl_b200.implementations.linear_layer import linear_layer

        return linear_layer(x, w_gate_up, None, activation="swiglu")

    @staticmethod
    def add_rms_norm(x, residual, w, eps):
        """(rms_norm(x + residual), x + residual) in one kernel."""
        from kernl_b200.implementations.layer_norm import layer_norm

        return layer_norm(x, w, None, eps, use_rms_norm=True, residual=residual)

    @staticmethod
    def rope_kv_write(qkv, k_cache, v_cache, cos, sin, pos, batch, seq):
        from kernl_b200.implementations.rope import rope_kv_write

        return rope_kv_write(qkv, k_cache, v_cache, cos, sin, pos, batch, seq)

    @staticmethod
    def attention_prefill(q, k, v, sm_scale):
        from kernl_b200.implementations.attention import attention_forward

        return attention_forward(q, k, v, torch.empty_like(q), sm_scale, True, None)

    @staticmethod
    def attention_decode(q, k, v, sm_scale, mask, kv_len):
        """One query row against the filled part of the cache: `kv_len` (device int64) keys are
        streamed, the slots behind them are never touched (no mask needed)."""
        from kernl_b200.implementations.attention_skinny import skinny_attention_forward

        return skinny_attention_forward(q, k, v, torch.empty_like(q), sm_scale, False, None, kv_len=kv_len)


def _seeded(shape, std, seed, device, dtype):
    """N(0, std) tensor that is identical on every rank (same seed, same generator device)."""
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding on interleaved pairs (x[..., 2i], x[..., 2i+1]) as in the reference's
    experimental kernels (experimental/llama-v2/kernel/pytorch_reference.py:37-80).
    x: [B, S, H, D]; cos/sin: [S, D/2] (or [B, S, D/2])."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    x0, x1 = xf[..., 0], xf[..., 1]
    c = cos.reshape(*cos.shape[:-1], 1, cos.shape[-1]) if cos.dim() == 2 else cos.unsqueeze(-2)
    s = sin.reshape(*sin.shape[:-1], 1, sin.shape[-1]) if sin.dim() == 2 else sin.unsqueeze(-2)
    out = torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)
    return out.reshape(x.shape).to(x.dtype)


class LlamaTP:
    """One rank's shard of the decoder."""

    def __init__(self, cfg: LlamaConfig, rank: int = 0, world: int = 1, device="cuda", dtype=torch.bfloat16,
                 ops=None, comm=None, seed: int = 0, weight_device: Optional[str] = None):
        assert cfg.n_heads % world == 0 and cfg.ffn % (8 * world) == 0
        self.cfg, self.rank, self.world, self.device, self.dtype = cfg, rank, world, torch.device(device), dtype
        self.ops = ops if ops is not None else CudaOps()
        self.comm = comm if comm is not None else NcclAllReduce(world)
        self.heads_local = cfg.n_heads // world
        self.ffn_local = cfg.ffn // world
        wd = weight_device or device
        H, D, F = cfg.hidden, cfg.head_dim, cfg.ffn
        hl, fl = self.heads_local, self.ffn_local
        r0h, r0f = rank * hl * D, rank * fl

        def shard_rows(full, start, n):
            return full[start:start + n].to(self.device).contiguous()

        self.embed = _seeded((cfg.vocab, H), 0.02, seed * 1000 + 1, wd, dtype).to(self.device)
        self.lm_head = _seeded((cfg.vocab, H), 0.02, seed * 1000 + 2, wd, dtype).to(self.device)
        self.final_norm = torch.ones(H, dtype=dtype, device=self.device)
        self.layers = []
        for li in range(cfg.n_layers):
            s = seed * 1000 + 10 * (li + 1)
            wq = _seeded((cfg.n_heads * D, H), 0.02, s + 1, wd, dtype)
            wk = _seeded((cfg.n_heads * D, H), 0.02, s + 2, wd, dtype)
            wv = _seeded((cfg.n_heads * D, H), 0.02, s + 3, wd, dtype)
            wqkv = torch.cat([shard_rows(w, r0h, hl * D) for w in (wq, wk, wv)], dim=0).contiguous()
            del wq, wk, wv
            wo = _seeded((H, cfg.n_heads * D), 0.02, s + 4, wd, dtype)[:, r0h:r0h + hl * D].to(self.device).contiguous()
            wg = _seeded((F, H), 0.02, s + 5, wd, dtype)
            wu = _seeded((F, H), 0.02, s + 6, wd, dtype)
            wgu = interleave_gate_up(shard_rows(wg, r0f, fl), shard_rows(wu, r0f, fl))
            del wg, wu
            wdn = _seeded((H, F), 0.02, s + 7, wd, dtype)[:, r0f:r0f + fl].to(self.device).contiguous()
            self.layers.append({
                "wqkv": wqkv, "wo": wo, "wgu": wgu, "wdn": wdn,
                "norm1": torch.ones(H, dtype=dtype, device=self.device),
                "norm2": torch.ones(H, dtype=dtype, device=self.device),
            })
        half = D // 2
        inv_freq = 1.0 / (cfg.rope_base ** (torch.arange(0, half, dtype=torch.float32) / half))
        ang = torch.arange(cfg.max_seq, dtype=torch.float32)[:, None] * inv_freq[None, :]
        self.cos, self.sin = torch.cos(ang).to(self.device), torch.sin(ang).to(self.device)
        self.kcache = None
        self.vcache = None
        self.sm_scale = D ** -0.5
        self.overlap_prefill = True  # two half-batches on two streams when tensor parallel (see prefill)
        # SMs left free for the collective while the two halves overlap: the GEMMs of the prefill are
        # persistent (one CTA per SM for the whole launch), so without this an all-reduce that is ready
        # to run finds no SM until the other half's GEMM has ended. 24 goes with a collective limited to
        # 24 CTAs (NCCL_MAX_CTAS=24, set by the caller before the process group exists); measured at
        # TP = 4, prefill 8 x 2048: 66.7 ms with nothing reserved, 61.5 ms with 24 / 24. Two ranks exchange
        # less; there the setting did not move the result (101.7-106.0 ms with 16 or 24 SMs)
        self.overlap_reserved_sms = int(os.environ.get("KERNL_B200_TP_RESERVED_SMS", "16" if world <= 2 else "24"))
        self._streams = None
        self._prefill_out = {}

    # ------------------------------------------------------------------ cache / state
    def alloc_cache(self, batch: int):
        cfg = self.cfg
        shape = (cfg.n_layers, batch, self.heads_local, cfg.max_seq, cfg.head_dim)
        self.kcache = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.vcache = torch.zeros(shape, dtype=self.dtype, device=self.device)
        # additive length mask for decode: 0 for filled slots, -inf beyond
        self.len_mask = torch.full((1, 1, 1, cfg.max_seq), float("-inf"), dtype=self.dtype, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.kv_len = torch.zeros(1, dtype=torch.long, device=self.device)  # filled slots seen by decode attention
        self._slots = torch.arange(cfg.max_seq, device=self.device).reshape(1, 1, 1, cfg.max_seq)
        self._host_pos = 0  # host-side copy of the position, for the length checks

    # ------------------------------------------------------------------ blocks
    def _row_parallel(self, x2d, w, residual, next_norm):
        """x = residual + all_reduce(x2d · wᵀ) and h = rms_norm(x) · next_norm, the input of the next
        sub-block. The GEMM writes its partial into the communicator's buffer when it has one
        (peer-mapped memory); reduce, residual add and norm are then one kernel. Returns (x, h)."""
        buf = self.comm.partial_buffer(x2d.shape[0], w.shape[0], x2d.dtype, x2d.device)
        partial = self.ops.linear(x2d, w, out=buf) if buf is not None else self.ops.linear(x2d, w)
        return self.comm.reduce_add_norm(partial, residual, next_norm, self.cfg.eps, self.ops)

    def _mlp(self, layer, h, residual, next_norm):
        act = self.ops.gated_linear(h, layer["wgu"])
        return self._row_parallel(act, layer["wdn"], residual, next_norm)

    def _next_norm(self, li):
        return self.layers[li + 1]["norm1"] if li + 1 < len(self.layers) else self.final_norm

    def prefill(self, ids: torch.Tensor, return_hidden: bool = False) -> torch.Tensor:
        """ids [B, S] → logits [B, vocab] of the last position; fills the KV cache. With
        `return_hidden` the final-norm hidden states of ALL positions, [B, S, hidden], are returned
        instead (what a parity check of inner positions needs)."""
        cfg, hl, D = self.cfg, self.heads_local, self.cfg.head_dim
        B, S = ids.shape
        assert S <= cfg.max_seq, f"prompt of {S} tokens does not fit the cache (max_seq {cfg.max_seq})"
        if self.kcache is None or self.kcache.shape[1] != B:
            self.alloc_cache(B)
        # Tensor parallel on GPUs: the batch is cut into two halves that run on two streams, so that
        # the all-reduce of one half (64 of them per prefill, 67 MB each at the 7B shape) travels
        # while the other half computes. Every rank enqueues the same sequence of collectives.
        # (only for messages far above what the one-shot peer-memory kernel takes: its single buffer
        # cannot serve two streams at once, and small messages gain nothing from the overlap)
        halves = 2 if (self.world > 1 and self.device.type == "cuda" and B % 2 == 0 and not return_hidden
                       and self.overlap_prefill and (B // 2) * S * cfg.hidden * 2 >= (8 << 20)) else 1
        if halves == 1:
            gen = self._prefill_rows(ids, 0, return_hidden)
            for _ in gen:
                pass
            h = self._prefill_out[0]
        else:
            main = torch.cuda.current_stream(self.device)
            if self._streams is None:
                self._streams = [torch.cuda.Stream(self.device) for _ in range(halves)]
            nb = B // halves
            gens = [self._prefill_rows(ids[i * nb:(i + 1) * nb], i * nb, False) for i in range(halves)]
            for st in self._streams:
                st.wait_stream(main)
            live = list(range(halves))
            lib = None
            if self.overlap_reserved_sms > 0:
                from kernl_b200 import _lib

                lib = _lib.load()
                sms = torch.cuda.get_device_properties(self.device).multi_processor_count
                lib.kb_gemm_sm_limit(max(2, sms - self.overlap_reserved_sms))
            try:
                while live:
                    for i in list(live):
                        with torch.cuda.stream(self._streams[i]):
                            try:
                                next(gens[i])
                            except StopIteration:
                                live.remove(i)
            finally:
                if lib is not None:
                    lib.kb_gemm_sm_limit(0)
            for i, st in enumerate(self._streams):
                main.wait_stream(st)
                self._prefill_out[i * nb].record_stream(main)
            h = torch.cat([self._prefill_out[i * nb] for i in range(halves)], dim=0)
        self._prefill_out = {}
        self.len_mask.fill_(float("-inf"))
        self.len_mask[..., :S] = 0
        self.pos.fill_(S)
        self.kv_len.fill_(S)
        self._host_pos = S
        if return_hidden:
            return h.reshape(B, S, cfg.hidden)
        return self.ops.linear(h, self.lm_head)  # h: final-norm hidden state of the last position of every sequence

    def _prefill_rows(self, ids: torch.Tensor, b0: int, return_hidden: bool):
        """The layer loop of the prefill for the sequences [b0, b0 + len(ids)) of the batch, written as
        a generator that yields after every collective, so that two parts of a batch can take turns.
        Leaves the final-norm hidden states (all positions, or the last one per sequence) in
        `self._prefill_out[b0]`."""
        cfg, hl, D = self.cfg, self.heads_local, self.cfg.head_dim
        B, S = ids.shape
        rows = slice(b0, b0 + B)
        x = self.embed.index_select(0, ids.reshape(-1)).reshape(B * S, cfg.hidden)
        h = self.ops.rms_norm(x, self.layers[0]["norm1"], cfg.eps)
        for li, layer in enumerate(self.layers):
            qkv = self.ops.linear(h, layer["wqkv"])
            # rotate q and k, write k and v into the cache at positions 0..S-1: one kernel
            q = self.ops.rope_kv_write(qkv, self.kcache[li, rows], self.vcache[li, rows], self.cos, self.sin, 0, B, S)
            attn = self.ops.attention_prefill(q.transpose(1, 2), self.kcache[li, rows, :, :S], self.vcache[li, rows, :, :S],
                                              self.sm_scale)  # [B, hl, S, D]
            attn2d = attn.transpose(1, 2).reshape(B * S, hl * D)
            x, h = self._row_parallel(attn2d, layer["wo"], x, layer["norm2"])
            yield
            x, h = self._mlp(layer, h, x, self._next_norm(li))
            yield
        if return_hidden:
            self._prefill_out[b0] = h
        else:
            self._prefill_out[b0] = h.reshape(B, S, cfg.hidden)[:, -1].contiguous()  # already through the final norm

    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] → logits [B, vocab]; appends one position to the cache. Every shape is static
        and the position lives on the device, so the step can be captured in one CUDA graph."""
        cfg, hl, D = self.cfg, self.heads_local, self.cfg.head_dim
        B = tokens.shape[0]
        x = self.embed.index_select(0, tokens)
        self.kv_len.add_(1)  # this step's token becomes the last of the keys
        if getattr(self.ops, "needs_len_mask", True):
            # open the slot of this position in the length mask. Written as a comparison against the
            # device-side position, so that a position at or beyond max_seq changes nothing instead
            # of indexing out of range (the callers check the length on the host as well).
            self.len_mask.masked_fill_(self._slots == self.pos, 0.0)
        h = self.ops.rms_norm(x, self.layers[0]["norm1"], cfg.eps)
        for li, layer in enumerate(self.layers):
            qkv = self.ops.linear(h, layer["wqkv"])
            q = self.ops.rope_kv_write(qkv, self.kcache[li], self.vcache[li], self.cos, self.sin, self.pos, B, 1)
            attn = self.ops.attention_decode(q.transpose(1, 2), self.kcache[li], self.vcache[li],
                                             self.sm_scale, self.len_mask, self.kv_len)  # [B, hl, 1, D]
            x, h = self._row_parallel(attn.reshape(B, hl * D), layer["wo"], x, layer["norm2"])
            x, h = self._mlp(layer, h, x, self._next_norm(li))
        self.pos.add_(1)
        return self.ops.linear(h, self.lm_head)

    def capture_decode(self, tokens: torch.Tensor):
        """Capture one decode step in a CUDA graph (after the prefill). Returns (replay, static_tok,
        static_next): copy the current tokens into `static_tok`, call `replay()`, read the greedy
        next tokens from `static_next`. The warm-up step and the capture advance the position and
        write cache slots; that state is restored here and the real steps overwrite the slots."""
        assert self._host_pos + 1 <= self.cfg.max_seq, "no free cache slot left for the capture's warm-up step"
        static_tok = tokens.clone()
        saved = (self.pos.clone(), self.len_mask.clone(), self.kv_len.clone())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.decode_step(static_tok)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            static_next = self.decode_step(static_tok).float().argmax(-1)
        self.pos.copy_(saved[0])
        self.len_mask.copy_(saved[1])
        self.kv_len.copy_(saved[2])
        self._decode_graph = graph  # keep the graph alive
        return graph.replay, static_tok, static_next

    def generate(self, ids: torch.Tensor, steps: int, use_cuda_graph: bool = True) -> torch.Tensor:
        """Greedy decoding: prefill, then `steps` tokens. Returns [B, steps] token ids. The argmax
        stays on the device, so no step waits for the host."""
        assert ids.shape[1] + max(steps - 1, 1) <= self.cfg.max_seq, (
            f"prompt {ids.shape[1]} + {steps} generated tokens exceed max_seq {self.cfg.max_seq}")
        logits = self.prefill(ids)
        tok = logits.float().argmax(-1)
        out = [tok]
        if use_cuda_graph and self.device.type == "cuda" and steps > 2:
            replay, static_tok, static_next = self.capture_decode(tok)
            for _ in range(steps - 1):
                static_tok.copy_(out[-1])
                replay()
                out.append(static_next.clone())
        else:
            for _ in range(steps - 1):
                out.append(self.decode_step(out[-1]).float().argmax(-1))
        self._host_pos += steps - 1
        tokens = torch.stack(out, dim=1)
        if self.device.type == "cuda":
            # a bounded device-side wait that expired makes later kernels skip their work: surface
            # it here rather than return tokens computed from stale buffers
            from kernl_b200 import _lib

            with torch.cuda.device(self.device):
                _lib.device_status()
        return tokens
