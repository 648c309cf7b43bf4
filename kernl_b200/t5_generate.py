"""T5 encoder-decoder inference on the kernl_b200 ops: encode once, then greedy decoding with a
static-shape KV cache so that one CUDA graph serves every decode step.

This is the host side of the baseline's fourth config (T5-base shape: 12+12 layers, d_model 768,
12 heads of 64, d_ff 3072 ReLU, RMS-style LayerNorm, 32 relative-position buckets). The weights and
the relative-position bias tables are taken from a Hugging Face `T5ForConditionalGeneration`
(its `compute_bias` is called once at set-up); everything per token runs on the library's
kernels: RMSNorm (kb_norm_fwd), all projections and the feed-forward (kb_linear_fwd, ReLU fused),
encoder self-attention with the position bias as additive mask (kb_attention_fwd), decoder self- and
cross-attention for one query row (kb_attention_decode_fwd, bias and length mask in-kernel).

The reference reaches the same model through TorchDynamo graphs of `generate` (one graph per
sequence length, tutorial/t5 e2e.ipynb) and sends the masked one-row attention of the decoder to
eager PyTorch (src/kernl/optimizer/attention.py:48-49); here the decode step is shape-static instead:
attention always covers the whole cache and an additive mask hides the unused slots.
"""
from typing import Optional

import torch

from kernl_b200.implementations.attention import attention_forward
from kernl_b200.implementations.attention_skinny import skinny_attention_forward
from kernl_b200.implementations.layer_norm import layer_norm
from kernl_b200.implementations.rope import rope_kv_write
from kernl_b200.implementations.linear_layer import linear_layer


def _w(t: torch.Tensor, device, dtype) -> torch.Tensor:
    return t.detach().to(device=device, dtype=dtype).contiguous()


class T5Kernl:
    def __init__(self, hf_model, device="cuda", dtype=torch.float16, max_new_tokens: int = 128):
        cfg = hf_model.config
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.H, self.Dh, self.dm = cfg.num_heads, cfg.d_kv, cfg.d_model
        self.eps = cfg.layer_norm_epsilon
        self.max_len = max_new_tokens + 1
        start = getattr(cfg, "decoder_start_token_id", None)
        self.start_token = start if start is not None else 0
        self.tied = bool(getattr(cfg, "tie_word_embeddings", True))
        assert cfg.feed_forward_proj == "relu", "only the ReLU feed-forward variant is wired up"
        d, dt = self.device, dtype
        self.embed = _w(hf_model.shared.weight, d, dt)
        self.lm_head = _w(hf_model.lm_head.weight, d, dt)

        def attn_weights(a):
            return {"qkv": torch.cat([_w(a.q.weight, d, dt), _w(a.k.weight, d, dt), _w(a.v.weight, d, dt)], dim=0).contiguous(),
                    "q": _w(a.q.weight, d, dt), "kv": torch.cat([_w(a.k.weight, d, dt), _w(a.v.weight, d, dt)], dim=0).contiguous(),
                    "o": _w(a.o.weight, d, dt)}

        self.enc_layers = []
        for blk in hf_model.encoder.block:
            ff = blk.layer[1].DenseReluDense
            self.enc_layers.append({"ln1": _w(blk.layer[0].layer_norm.weight, d, dt), "attn": attn_weights(blk.layer[0].SelfAttention),
                                    "ln2": _w(blk.layer[1].layer_norm.weight, d, dt), "wi": _w(ff.wi.weight, d, dt), "wo": _w(ff.wo.weight, d, dt)})
        self.enc_final_ln = _w(hf_model.encoder.final_layer_norm.weight, d, dt)
        self.dec_layers = []
        for blk in hf_model.decoder.block:
            ff = blk.layer[2].DenseReluDense
            self.dec_layers.append({"ln1": _w(blk.layer[0].layer_norm.weight, d, dt), "self": attn_weights(blk.layer[0].SelfAttention),
                                    "ln2": _w(blk.layer[1].layer_norm.weight, d, dt), "cross": attn_weights(blk.layer[1].EncDecAttention),
                                    "ln3": _w(blk.layer[2].layer_norm.weight, d, dt), "wi": _w(ff.wi.weight, d, dt), "wo": _w(ff.wo.weight, d, dt)})
        self.dec_final_ln = _w(hf_model.decoder.final_layer_norm.weight, d, dt)
        self._enc_bias_module = hf_model.encoder.block[0].layer[0].SelfAttention
        with torch.no_grad():
            # decoder self-attention bias for every (query position, key position): [H, L, L]
            dec_bias = hf_model.decoder.block[0].layer[0].SelfAttention.compute_bias(self.max_len, self.max_len)[0]
        self.dec_bias = dec_bias.to(device=d, dtype=dt).permute(1, 0, 2).contiguous()  # [L(query), H, L(key)]
        self._enc_bias_cache = {}
        # T5 has no rotary embedding: identity rotation tables for the shared cache-write kernel
        self.rot_cos = torch.ones((self.max_len, self.Dh // 2), dtype=torch.float32, device=d)
        self.rot_sin = torch.zeros((self.max_len, self.Dh // 2), dtype=torch.float32, device=d)

    # ------------------------------------------------------------------ helpers
    def _rms(self, x, w):
        return layer_norm(x, w, None, self.eps, use_rms_norm=True)

    def _add_rms(self, y, residual, w):
        """(rms_norm(y + residual) * w, y + residual) in one kernel."""
        return layer_norm(y, w, None, self.eps, use_rms_norm=True, residual=residual)

    def _enc_bias(self, S: int) -> torch.Tensor:
        if S not in self._enc_bias_cache:
            with torch.no_grad():
                bias = self._enc_bias_module.compute_bias(S, S)  # [1, H, S, S] on the module's device
            self._enc_bias_cache[S] = bias.to(device=self.device, dtype=self.dtype).contiguous()
        return self._enc_bias_cache[S]

    # ------------------------------------------------------------------ encoder
    def encode(self, ids: torch.Tensor) -> torch.Tensor:
        B, S = ids.shape
        H, Dh = self.H, self.Dh
        x = self.embed.index_select(0, ids.reshape(-1))
        bias = self._enc_bias(S)
        h = self._rms(x, self.enc_layers[0]["ln1"])
        for li, L in enumerate(self.enc_layers):
            qkv = linear_layer(h, L["attn"]["qkv"], None).reshape(B, S, 3, H, Dh)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))  # [B, H, S, Dh] views
            o = attention_forward(q, k, v, torch.empty_like(q), 1.0, False, bias)
            h, x = self._add_rms(linear_layer(o.transpose(1, 2).reshape(B * S, H * Dh), L["attn"]["o"], None), x, L["ln2"])
            nxt = self.enc_layers[li + 1]["ln1"] if li + 1 < len(self.enc_layers) else self.enc_final_ln
            h, x = self._add_rms(linear_layer(linear_layer(h, L["wi"], None, "relu"), L["wo"], None), x, nxt)
        return h.reshape(B, S, self.dm)  # already through the final norm

    # ------------------------------------------------------------------ decoder
    def start(self, enc_out: torch.Tensor):
        """Allocate the caches for this batch and project the encoder output once per layer."""
        B, S, _ = enc_out.shape
        H, Dh, d, dt = self.H, self.Dh, self.device, self.dtype
        nl = len(self.dec_layers)
        e2 = enc_out.reshape(B * S, self.dm)
        if getattr(self, "_state_shape", None) == (B, S):
            # same shapes as the previous request: keep the buffers (and the captured decode graph
            # that reads them), refill them in place
            self.len_mask.fill_(float("-inf"))
            self.pos.zero_()
            for li, L in enumerate(self.dec_layers):
                kv = linear_layer(e2, L["cross"]["kv"], None).reshape(B, S, 2, H, Dh)
                self.cross_k[li].copy_(kv[:, :, 0].transpose(1, 2))
                self.cross_v[li].copy_(kv[:, :, 1].transpose(1, 2))
            return
        self._state_shape = (B, S)
        self._graph = None
        self.kcache = torch.zeros((nl, B, H, self.max_len, Dh), dtype=dt, device=d)
        self.vcache = torch.zeros((nl, B, H, self.max_len, Dh), dtype=dt, device=d)
        self.len_mask = torch.full((1, 1, 1, self.max_len), float("-inf"), dtype=dt, device=d)
        self.pos = torch.zeros(1, dtype=torch.long, device=d)
        self._slots = torch.arange(self.max_len, device=d).reshape(1, 1, 1, self.max_len)
        self.cross_k, self.cross_v = [], []
        for L in self.dec_layers:
            kv = linear_layer(e2, L["cross"]["kv"], None).reshape(B, S, 2, H, Dh)
            self.cross_k.append(kv[:, :, 0].transpose(1, 2).contiguous())
            self.cross_v.append(kv[:, :, 1].transpose(1, 2).contiguous())

    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] → logits [B, vocab] for the next position. Static shapes; the position is a
        device tensor."""
        B = tokens.shape[0]
        H, Dh = self.H, self.Dh
        x = self.embed.index_select(0, tokens)
        # open this position's slot; a comparison, so that no position can index out of range
        self.len_mask.masked_fill_(self._slots == self.pos, 0.0)
        # bias row of the current query position + the length mask: [1, H, 1, L]
        self_mask = (self.dec_bias.index_select(0, self.pos).reshape(1, H, 1, self.max_len) + self.len_mask).contiguous()
        # The residual stream is carried as (x, h): every "x + sublayer" and the norm that follows it
        # are one kernel, and the k/v of the new token go into the cache through the same kernel that
        # the Llama decoder uses for rotary + cache write (with cos = 1, sin = 0 it only moves data).
        h = self._rms(x, self.dec_layers[0]["ln1"])
        n_layers = len(self.dec_layers)
        for li, L in enumerate(self.dec_layers):
            qkv = linear_layer(h, L["self"]["qkv"], None)
            q = rope_kv_write(qkv, self.kcache[li], self.vcache[li], self.rot_cos, self.rot_sin, self.pos, B, 1)
            q = q.transpose(1, 2)  # [B, H, 1, Dh] view
            o = skinny_attention_forward(q, self.kcache[li], self.vcache[li], torch.empty((B, H, 1, Dh), dtype=q.dtype, device=q.device),
                                         1.0, False, self_mask)
            h, x = self._add_rms(linear_layer(o.reshape(B, H * Dh), L["self"]["o"], None), x, L["ln2"])
            q = linear_layer(h, L["cross"]["q"], None).reshape(B, H, 1, Dh)
            o = skinny_attention_forward(q, self.cross_k[li], self.cross_v[li], torch.empty_like(q), 1.0, False, None)
            h, x = self._add_rms(linear_layer(o.reshape(B, H * Dh), L["cross"]["o"], None), x, L["ln3"])
            nxt = self.dec_layers[li + 1]["ln1"] if li + 1 < n_layers else self.dec_final_ln
            h, x = self._add_rms(linear_layer(linear_layer(h, L["wi"], None, "relu"), L["wo"], None), x, nxt)
        self.pos.add_(1)
        x = h  # already through the final norm
        if self.tied:
            x = x * (self.dm ** -0.5)
        return linear_layer(x, self.lm_head, None)

    def generate(self, ids: torch.Tensor, steps: Optional[int] = None, use_cuda_graph: bool = True) -> torch.Tensor:
        """Greedy decoding of `steps` tokens (default: the configured maximum). Returns [B, steps]."""
        steps = steps if steps is not None else self.max_len - 1
        assert steps <= self.max_len - 1
        B = ids.shape[0]
        self.start(self.encode(ids))
        tok = torch.full((B,), self.start_token, dtype=torch.long, device=self.device)
        out = []
        if use_cuda_graph and steps > 2:
            if getattr(self, "_graph", None) is None:
                static_tok = tok.clone()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.decode_step(static_tok)  # warm-up (writes slot 0, which the first real step rewrites)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    static_next = self.decode_step(static_tok).float().argmax(-1)
                self.pos.zero_()
                self.len_mask.fill_(float("-inf"))
                self._graph = (graph, static_tok, static_next)  # reused while the shapes stay the same
            graph, static_tok, static_next = self._graph
            for _ in range(steps):
                static_tok.copy_(tok)
                graph.replay()
                tok = static_next.clone()
                out.append(tok)
        else:
            for _ in range(steps):
                tok = self.decode_step(tok).float().argmax(-1)
                out.append(tok)
        tokens = torch.stack(out, dim=1)
        if self.device.type == "cuda":
            # kernels skip their work after a bounded device-side wait has expired: report that
            # here rather than hand back tokens computed from stale buffers
            from kernl_b200 import _lib

            with torch.cuda.device(self.device):
                _lib.device_status()
        return tokens
