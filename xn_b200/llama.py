"""A Llama-style decoder whose every linear runs through the quantized matmul library.

Mirrors the structure of the reference's model (xn-core/src/models/llama.rs:130-330: pre-norm blocks,
q/k/v/o projections with grouped-query attention and RoPE, SwiGLU MLP, final norm, LM head), with all
linears held as GGUF-quantized device weights (``QCudaTensor``) instead of dense ``Linear``s, the way
``BackendQ::linear_load`` substitutes them (lib.rs:141-156).

Tensor parallelism over ``world`` ranks (one process per GPU):
  * q/k/v are N-sharded with rows grouped per rank by head, so attention and the KV cache are
    head-sharded and the fused ``[q_r; k_r; v_r]`` projection needs no exchange;
  * gate/up are N-sharded with rows grouped per rank, SwiGLU is applied to the local slice (gate and up
    are only consumed through ``silu(gate) * up``, llama.rs:258-265);
  * o_proj and down_proj are K-sharded (each rank multiplies its own slice of the input with the matching
    column blocks of the weight; a K-shard is whole quantization blocks, so its block dots are exactly
    the unsharded ones): two exchanges per layer, each done by the matmul kernel itself, which stores
    its summand into every rank's buffer; the next residual-add + RMSNorm adds the summands;
  * the LM head is N-sharded and its output columns are gathered the same way.

Prefill runs RMSNorm, RoPE and attention as torch ops. A decode step uses the library's fused operators
between the linears (residual-add + RMSNorm, RoPE + KV-cache store, single-query attention, SwiGLU), so
one layer is ten launches and the whole step is one CUDA graph.
"""
from __future__ import annotations

import os

import dataclasses
from typing import Optional

import torch
import torch.nn.functional as F

from . import decoder_ops as ops
from .dtypes import GgmlDType
from .parallel import PeerGather
from .quantized import QCudaTensor, init


@dataclasses.dataclass
class LlamaConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 32000
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    linear_dtype: GgmlDType = GgmlDType.Q4K
    head_dtype: GgmlDType = GgmlDType.Q6K

    @classmethod
    def llama_7b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=512)

    def weight_bytes_per_step(self) -> int:
        """GGUF bytes of all linears, each read once per decode step."""
        ld, hd = self.linear_dtype, self.head_dtype
        per_layer = (ld.row_bytes(self.d_model) * ((self.n_heads + 2 * self.n_kv_heads) * self.head_dim + self.d_model + 2 * self.ffn)
                     + ld.row_bytes(self.ffn) * self.d_model)
        return self.n_layers * per_layer + hd.row_bytes(self.d_model) * self.vocab


def _dense(shape, std, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std


class _Layer:
    __slots__ = ("wqkv", "wo", "wgu", "wdown", "norm1", "norm2", "k_cache", "v_cache")


class QLlama:
    """Random-init weights (N(0, 0.02), quantized on the device with the reference's quantizers), a
    KV cache of ``max_seq`` positions for ``batch`` sequences, prefill and CUDA-graphed decode."""

    def __init__(self, cfg: LlamaConfig, device: torch.device, batch: int = 1, max_seq: int = 1024, rank: int = 0, world: int = 1,
                 group=None, seed: int = 0, max_prefill_rows: int = 512, fused_decode: bool = True, fused_norm: Optional[bool] = None, fused_rope: bool = True):
        if cfg.n_kv_heads % world or cfg.n_heads % world or cfg.ffn % world or cfg.vocab % world or cfg.d_model % world:
            raise ValueError(f"config does not divide over {world} ranks")
        init(device)
        self.cfg, self.device, self.batch, self.max_seq, self.rank, self.world = cfg, device, batch, max_seq, rank, world
        self.hl, self.kvl = cfg.n_heads // world, cfg.n_kv_heads // world
        self.fused_decode = fused_decode and cfg.head_dim == 128
        # One-row decode: residual add + RMSNorm in the prologue of the matvec that follows (same bits either way): two launches
        # fewer per layer (690 against 661 tok/s on one GPU), and sharded it is where the exchange of the row-parallel linears is
        # awaited, off the producing kernel's critical path. XN_FUSED_NORM=0/1 overrides the default for measurements.
        if fused_norm is None:
            env = os.environ.get("XN_FUSED_NORM")
            fused_norm = (env == "1") if env in ("0", "1") else True
        self.fused_norm = fused_norm
        self.fused_rope = fused_rope
        c, r, G, hd = cfg, rank, world, cfg.head_dim

        def rows(w, per):  # this rank's block of `per` consecutive rows
            return w[r * per:(r + 1) * per]

        self.layers = []
        for li in range(c.n_layers):
            s0 = seed * 1_000_003 + li * 16
            L = _Layer()
            wq = rows(_dense((c.n_heads * hd, c.d_model), 0.02, s0 + 0, device), self.hl * hd)
            wk = rows(_dense((c.n_kv_heads * hd, c.d_model), 0.02, s0 + 1, device), self.kvl * hd)
            wv = rows(_dense((c.n_kv_heads * hd, c.d_model), 0.02, s0 + 2, device), self.kvl * hd)
            L.wqkv = QCudaTensor.from_dense(torch.cat([wq, wk, wv]), c.linear_dtype)
            del wq, wk, wv
            L.wo = self._kshard(_dense((c.d_model, c.n_heads * hd), 0.02, s0 + 3, device), c.linear_dtype)
            wg = rows(_dense((c.ffn, c.d_model), 0.02, s0 + 4, device), c.ffn // G)
            wu = rows(_dense((c.ffn, c.d_model), 0.02, s0 + 5, device), c.ffn // G)
            L.wgu = QCudaTensor.from_dense(torch.cat([wg, wu]), c.linear_dtype)
            del wg, wu
            L.wdown = self._kshard(_dense((c.d_model, c.ffn), 0.02, s0 + 6, device), c.linear_dtype)
            L.norm1 = torch.ones(c.d_model, device=device)
            L.norm2 = torch.ones(c.d_model, device=device)
            L.k_cache = torch.zeros((batch, self.kvl, max_seq, hd), device=device, dtype=torch.bfloat16)
            L.v_cache = torch.zeros_like(L.k_cache)
            self.layers.append(L)
        self.norm = torch.ones(c.d_model, device=device)
        self.embed = _dense((c.vocab, c.d_model), 0.02, seed * 1_000_003 + 900_001, device).to(torch.bfloat16)
        self.lm_head = self._shard(_dense((c.vocab, c.d_model), 0.02, seed * 1_000_003 + 900_002, device), c.head_dtype)

        inv = 1.0 / (c.rope_theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
        ang = torch.arange(max_seq, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()  # [max_seq, hd/2]

        self.pg: Optional[PeerGather] = None
        if world > 1:
            rows_max = max(batch, max_prefill_rows)
            self.pg = PeerGather(device, rank, world, slot_elems=max(rows_max * c.d_model * world, batch * c.vocab), nslots=3, group=group)
            self._gathers_per_step = 2 * c.n_layers + 1
        # decode-step state, all on the device so a captured graph can be replayed
        self.pos = torch.zeros(1, device=device, dtype=torch.int64)
        self.tokens = torch.zeros(batch, device=device, dtype=torch.int64)
        self._graph = None
        f32 = dict(device=device, dtype=torch.float32)
        self._x = torch.zeros((batch, c.d_model), **f32)       # residual stream of the decode step
        self._x2 = torch.zeros((batch, c.d_model), **f32)      # its second buffer: a fused norm + matvec reads one and writes the other
        self._logits = torch.zeros((batch, c.vocab), **f32) if world == 1 else None
        self._xn = torch.zeros((batch, c.d_model), **f32)
        self._qkv = torch.zeros((batch, (self.hl + 2 * self.kvl) * hd), **f32)
        self._q = torch.zeros((batch, self.hl, hd), **f32)
        self._a = torch.zeros((batch, self.hl * hd), **f32)
        self._gu = torch.zeros((batch, 2 * c.ffn // G), **f32)
        self._h = torch.zeros((batch, c.ffn // G), **f32)
        self._o = torch.zeros((batch, c.d_model), **f32)
        self._dn = torch.zeros((batch, c.d_model), **f32)
        # The norm's and the SwiGLU's outputs are only ever read by quantized linears, so their producers can write
        # them as activation images (quantized once). That pays wherever the matmul would otherwise launch its own
        # quantizer kernel: batches above one, and k above 4096. The one-row k <= 4096 decode kernel quantizes in
        # its prologue, hidden behind its weight prefetch, and is better left alone.
        def wants_image(k):
            return batch <= 16 and k % 256 == 0 and (batch > 1 or k > 4096)
        # Batches of 2..64 rows on Q4_K linears: the images are written in the integer tensor-core kernel's own layout, and each such
        # linear is one kernel instead of two (XN_OPERAND_IMAGES=0/1 for measurements).
        env = os.environ.get("XN_OPERAND_IMAGES")
        operand = (env == "1" if env in ("0", "1") else True) and 2 <= batch <= 64 and c.linear_dtype == GgmlDType.Q4K and world == 1
        def image(k):
            if operand and k % 256 == 0:
                return ops.OperandImage(batch, k, device)
            return ops.ActImage.for_weight(c.linear_dtype, batch, k, device) if wants_image(k) else None
        self._xn_img = image(c.d_model)
        self._h_img = image(c.ffn // G)
        if isinstance(self._xn_img, ops.OperandImage):   # the LM head is not an integer tensor-core weight: it keeps a planar image, or float rows
            self._head_img = ops.ActImage.for_weight(c.head_dtype, batch, c.d_model, device) if wants_image(c.d_model) else None
        else:
            self._head_img = self._xn_img if c.head_dtype.vec_dot_type == c.linear_dtype.vec_dot_type else None

        for L in self.layers:   # scratch is sized once, before any capture
            for w in (L.wqkv, L.wo, L.wgu, L.wdown):
                w.workspace(max(batch, max_prefill_rows))
        self.lm_head.workspace(batch)

    # -- pieces ----------------------------------------------------------------------------------
    def _shard(self, dense: torch.Tensor, dt: GgmlDType) -> QCudaTensor:
        """Quantize and keep this rank's rows of an N-sharded linear (quantization is per row, so slicing first is exact)."""
        from .quantized import quantize_weight
        n, k = dense.shape
        per = n // self.world
        blocks = quantize_weight(dense[self.rank * per:(self.rank + 1) * per], dt)
        return QCudaTensor.from_device_rows(dt, blocks, n, k, self.rank * per, per)

    def _kshard(self, dense: torch.Tensor, dt: GgmlDType) -> QCudaTensor:
        """This rank's column blocks of a row-parallel linear: a whole-N weight over K/world inputs."""
        per = dense.shape[1] // self.world
        if per % dt.block_size:
            raise ValueError(f"k = {dense.shape[1]} does not split into {self.world} runs of whole {dt.name} blocks")
        return QCudaTensor.from_dense(dense[:, self.rank * per:(self.rank + 1) * per].contiguous(), dt)

    def _linear_gathered(self, w: QCudaTensor, x: torch.Tensor) -> torch.Tensor:
        """N-sharded linear, output columns gathered on every rank."""
        return w.matmul_t(x) if self.pg is None else self.pg.matmul_t(w, x, slot=self._slot())

    def _linear_parts(self, w: QCudaTensor, x_local: torch.Tensor, out: Optional[torch.Tensor] = None, defer: bool = False) -> torch.Tensor:
        """K-sharded linear on this rank's input slice: ``(.., world * n)``, the ranks' summands side by side. ``defer``: the
        kernel publishes its columns and retires without awaiting the peers'; the consumer of the result awaits them."""
        if self.pg is None:
            return w.matmul_t(x_local, out=out)
        self.pg.set_deferred(defer)
        try:
            return self.pg.matmul_t(w, x_local, slot=self._slot(), parts=True)
        finally:
            self.pg.set_deferred(False)

    def _sum_parts(self, parts: torch.Tensor) -> torch.Tensor:
        return parts if self.world == 1 else parts.view(*parts.shape[:-1], self.world, -1).sum(-2)

    def _slot(self) -> int:
        # three slots in rotation; a step's last exchange must not land on the slot its first one uses
        i = self._gather_idx
        self._gather_idx = (i + 1) % self._gathers_per_step
        s = i % 3
        if i == self._gathers_per_step - 1 and s == 0:
            s = 1 if (i - 1) % 3 != 1 else 2
        return s

    def _rms(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.cfg.rms_eps) * w

    @staticmethod
    def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        # x [B, H, S, hd]; cos / sin [S, hd/2]; rotate-half convention
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    def _block(self, L: _Layer, x: torch.Tensor, pos_idx: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """x [B, S, d]; pos_idx [S] int64 positions of these tokens; mask broadcastable to [B, H, S, max_seq]."""
        c, hd = self.cfg, self.cfg.head_dim
        B, S, _ = x.shape
        qkv = L.wqkv.matmul_t(self._rms(x, L.norm1))
        q, k, v = qkv.split([self.hl * hd, self.kvl * hd, self.kvl * hd], dim=-1)
        q = q.view(B, S, self.hl, hd).transpose(1, 2)
        k = k.view(B, S, self.kvl, hd).transpose(1, 2)
        v = v.view(B, S, self.kvl, hd).transpose(1, 2)
        cos, sin = self.cos.index_select(0, pos_idx), self.sin.index_select(0, pos_idx)
        q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
        L.k_cache.index_copy_(2, pos_idx, k.to(torch.bfloat16))
        L.v_cache.index_copy_(2, pos_idx, v.to(torch.bfloat16))
        a = F.scaled_dot_product_attention(q.to(torch.bfloat16), L.k_cache, L.v_cache, attn_mask=mask, enable_gqa=True)
        a = a.transpose(1, 2).reshape(B, S, self.hl * hd).float()
        x = x + self._sum_parts(self._linear_parts(L.wo, a))
        gu = L.wgu.matmul_t(self._rms(x, L.norm2))
        g, u = gu.split(c.ffn // self.world, dim=-1)
        x = x + self._sum_parts(self._linear_parts(L.wdown, F.silu(g) * u))
        return x

    def _forward(self, tokens: torch.Tensor, pos_idx: torch.Tensor) -> torch.Tensor:
        """tokens [B, S] -> logits of the last position [B, vocab]."""
        self._gather_idx = 0
        ar = torch.arange(self.max_seq, device=self.device)
        mask = (ar[None, :] <= pos_idx[:, None])[None, None]  # [1, 1, S, max_seq]: causal over the cache
        x = self.embed.index_select(0, tokens.reshape(-1)).view(*tokens.shape, -1).float()
        for L in self.layers:
            x = self._block(L, x, pos_idx, mask)
        x = self._rms(x[:, -1:, :], self.norm)
        logits = self._linear_gathered(self.lm_head, x).view(tokens.shape[0], -1)
        return logits if self.pg is None else logits.clone()   # out of the exchange slot before it is reused

    def _forward_decode(self) -> torch.Tensor:
        """One token per sequence (self.tokens at position self.pos) -> logits [B, vocab], fused operators."""
        c = self.cfg
        self._gather_idx = 0
        ops.embed_rows(self.embed, self.tokens, self._x)   # one plain launch: the step's barrier against the step before
        delta = None
        xi, hi = self._xn_img, self._h_img
        # one row: every linear's kernel is told which weight comes next, and asks for it to be brought into L2 as it finishes
        hint = (lambda w: w.hint_next()) if self.batch == 1 else (lambda w: None)
        # One row and rows of at most 4096 values: the residual add, the RMSNorm and the quantizer run in the prologue of the
        # matvec that consumes them (same bits as the separate kernels), which takes two launches out of every layer.
        fused = self.batch == 1 and self.fused_norm and self.layers[0].wqkv.supports_normed()
        cur, nxt = self._x, self._x2
        # sharded: the K-sharded linears leave their exchange un-awaited, the fused kernel that adds the summands awaits the
        # peers itself while its weight stream is already running
        defer = fused and self.pg is not None
        for li, L in enumerate(self.layers):
            hint(L.wo)
            if fused:
                L.wqkv.matvec_normed(cur, delta, L.norm1, c.rms_eps, nxt, self._qkv, await_comm=self.pg if (defer and delta is not None) else None)
                cur, nxt = nxt, cur
            else:
                ops.add_rmsnorm(cur, delta, L.norm1, c.rms_eps, None if xi else self._xn, xi)
                L.wqkv.matmul_t(xi or self._xn, out=self._qkv)
            if self.fused_rope:   # RoPE and the KV-cache store inside the attention kernel: one launch less per layer, same bits
                ops.rope_attn_decode(self._qkv, self.cos, self.sin, self.pos, L.k_cache, L.v_cache, self._a.view(self.batch, self.hl, c.head_dim), self.hl, self.kvl)
            else:
                ops.rope_kv_store(self._qkv, self.cos, self.sin, self.pos, self._q, L.k_cache, L.v_cache, self.hl, self.kvl)
                ops.attn_decode(self._q, L.k_cache, L.v_cache, self.pos, self._a.view(self.batch, self.hl, c.head_dim), self.hl, self.kvl)
            hint(L.wgu)
            o = self._linear_parts(L.wo, self._a, self._o, defer=defer)           # world summands per row when sharded
            hint(L.wdown)
            if fused:
                L.wgu.matvec_normed(cur, o, L.norm2, c.rms_eps, nxt, self._gu, await_comm=self.pg if defer else None)
                cur, nxt = nxt, cur
            else:
                ops.add_rmsnorm(cur, o, L.norm2, c.rms_eps, None if xi else self._xn, xi)
                L.wgu.matmul_t(xi or self._xn, out=self._gu)
            ops.swiglu(self._gu, None if hi else self._h, hi)
            hint(self.layers[li + 1].wqkv if li + 1 < len(self.layers) else self.lm_head)
            delta = self._linear_parts(L.wdown, hi or self._h, self._dn, defer=defer and li + 1 < len(self.layers))  # the last one feeds an unfused norm
        fi = self._head_img
        if fused and self.pg is None and self.lm_head.supports_normed():
            logits = self.lm_head.matvec_normed(cur, delta, self.norm, c.rms_eps, nxt, self._logits)
        else:
            ops.add_rmsnorm(cur, delta, self.norm, c.rms_eps, None if fi else self._xn, fi)
            logits = self._linear_gathered(self.lm_head, fi or self._xn)
        return logits if self.pg is None else logits.clone()   # out of the exchange slot before it is reused

    # -- public ----------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """prompt [B, S] token ids; fills the cache, sets the decode position, returns the last logits."""
        B, S = prompt.shape
        pos_idx = torch.arange(S, device=self.device)
        logits = self._forward(prompt, pos_idx)
        self.pos.fill_(S)
        self.tokens.copy_(logits.argmax(-1))
        return logits

    @torch.no_grad()
    def _decode_step(self) -> None:
        logits = self._forward_decode() if self.fused_decode else self._forward(self.tokens.view(-1, 1), self.pos)
        if self.fused_decode and logits.dtype is torch.float32 and logits.is_contiguous():
            ops.argmax_advance(logits, self.tokens, self.pos)   # greedy choice and position advance in one launch
        else:
            self.tokens.copy_(logits.argmax(-1))
            self.pos.add_(1)
        self.last_logits = logits

    @torch.no_grad()
    def capture_decode(self) -> None:
        """Record one decode step (all layers, LM head, greedy sampling, position advance) as a CUDA graph."""
        pos0, tok0 = self.pos.clone(), self.tokens.clone()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        from . import _lib
        with torch.cuda.stream(side):
            before = _lib.lib().xnq_launch_count()
            self._decode_step()   # warm-up outside the capture (lazy initialisations of torch's own kernels)
            self.launches_per_step = int(_lib.lib().xnq_launch_count() - before)   # the library's own kernels in one step
            self.pos.copy_(pos0); self.tokens.copy_(tok0)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                self._decode_step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.pos.copy_(pos0); self.tokens.copy_(tok0)
        self._graph = g

    def decode(self, steps: int) -> torch.Tensor:
        """Run `steps` greedy decode steps; returns the generated ids [B, steps]."""
        out = torch.empty((self.batch, steps), device=self.device, dtype=torch.int64)
        for i in range(steps):
            if self._graph is not None:
                self._graph.replay()
            else:
                self._decode_step()
            out[:, i] = self.tokens
        return out

    def close(self):
        if self.pg is not None:
            self.pg.close()
            self.pg = None



def dense_reference_logits(model: QLlama, tokens: torch.Tensor) -> torch.Tensor:
    """The same network evaluated with dense f32 matmuls on the DEQUANTIZED weights and f32 attention
    (single rank only): what the quantized path approximates up to activation-quantization error."""
    assert model.world == 1
    c, hd = model.cfg, model.cfg.head_dim
    B, S = tokens.shape
    x = model.embed.index_select(0, tokens.reshape(-1)).view(B, S, -1).float()
    pos = torch.arange(S, device=model.device)
    cos, sin = model.cos[:S], model.sin[:S]
    causal = torch.ones(S, S, device=model.device, dtype=torch.bool).tril()
    for L in model.layers:
        qkv = model._rms(x, L.norm1) @ L.wqkv.dequantize(torch.float32).T
        q, k, v = qkv.split([c.n_heads * hd, c.n_kv_heads * hd, c.n_kv_heads * hd], dim=-1)
        q = model._rope(q.view(B, S, c.n_heads, hd).transpose(1, 2), cos, sin)
        k = model._rope(k.view(B, S, c.n_kv_heads, hd).transpose(1, 2), cos, sin)
        v = v.view(B, S, c.n_kv_heads, hd).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=causal, enable_gqa=True)
        x = x + a.transpose(1, 2).reshape(B, S, -1) @ L.wo.dequantize(torch.float32).T
        g, u = (model._rms(x, L.norm2) @ L.wgu.dequantize(torch.float32).T).split(c.ffn, dim=-1)
        x = x + (F.silu(g) * u) @ L.wdown.dequantize(torch.float32).T
    return (model._rms(x[:, -1:, :], model.norm) @ model.lm_head.dequantize(torch.float32).T).view(B, -1)
