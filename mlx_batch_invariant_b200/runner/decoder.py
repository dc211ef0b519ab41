"""Llama-3-architecture decoder over the batch-invariant ops, sharded without reductions.

This is the whole-model caller the reference exercises through ``mlx_lm`` (harness/model_sweep.py:89-108
and harness/generate_bench.py:24-33 there): prefill a batch of prompts, then greedy-decode with a KV
cache, all linear / norm / attention math going through the four batch-invariant kernels.

Sharding (R ranks, one process per GPU) uses only dimensions that need no cross-GPU reduction:
  * every linear is column-parallel: rank r owns rows [r*N/R, (r+1)*N/R) of W[N, K] and produces
    the matching slice of the output features;
  * attention is sharded by KV head (each rank keeps the cache of its own heads);
  * the feature slices are joined by all-gather (3 per layer + 1 for the logits; the attention output
    projection is replicated, which is cheaper than a fourth gather).
Each output element is produced on exactly one GPU by the same K order as on one GPU, so logits are
bit-identical for every R and every batch size. RMSNorm, RoPE, residual adds, SwiGLU and argmax are
replicated or elementwise.
"""

from __future__ import annotations

import hashlib
import math
import os
import sys
from dataclasses import dataclass

import torch

from .. import kernels as K


@dataclass(frozen=True)
class DecoderConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    init_std: float = 0.02


LLAMA3_8B = DecoderConfig()

PUSH_TESTED_WORLDS = (2, 4, 8)  # world sizes at which the peer-memory all-gather has run on hardware
PUSH_PARTIALS_MAX = 256 << 20   # a matmul pushes its own output only while its split partials stay below this many bytes


class TorchGlue:
    """Framework-op versions of the elementwise glue (used by CPU stand-in backends in tests)."""

    def rope_append(self, qkv, cos, sin, pos0, B, T, hq, hkv, D, kc, vc):
        """qkv[B*T, (hq+2hkv)*D] -> rotated q[B, hq, T, D]; rotated k and v written into the caches at
        positions pos0 .. pos0+T-1 (pos0: int64 tensor of one element)."""
        x = qkv.reshape(B, T, hq + 2 * hkv, D).transpose(1, 2)
        pos = pos0 + torch.arange(T, device=qkv.device)
        c, s_ = cos.index_select(0, pos)[None, None], sin.index_select(0, pos)[None, None]

        def rot(t):
            tf = t.float()
            half = D // 2
            r = torch.cat([-tf[..., half:], tf[..., :half]], -1)
            return (tf * c + r * s_).to(t.dtype)

        kc[:B].index_copy_(2, pos, rot(x[:, hq:hq + hkv]))
        vc[:B].index_copy_(2, pos, x[:, hq + hkv:].contiguous())
        return rot(x[:, :hq]).contiguous()

    def swiglu(self, gu):
        f = gu.shape[1] // 2
        g = gu[:, :f].float()
        return (g * torch.sigmoid(g) * gu[:, f:].float()).to(gu.dtype)

    def add_rms_norm(self, x, delta, w, eps):
        """Residual add followed by the norm of the sum: returns (x + delta, rms_norm(x + delta))."""
        s = x + delta
        return s, self.rms_norm(s, w, eps)


class KernelBackend(TorchGlue):
    """The four batch-invariant ops plus the glue kernels. Tests of the sharding logic swap in a CPU stand-in."""

    def rope_append(self, qkv, cos, sin, pos0, B, T, hq, hkv, D, kc, vc):
        from .. import _lib
        q = torch.empty(B, hq, T, D, dtype=qkv.dtype, device=qkv.device)
        qkv = qkv.contiguous()
        _lib.check(_lib.load().bi_rope_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos0.data_ptr(), q.data_ptr(),
                                              kc.data_ptr(), vc.data_ptr(), B, T, hq, hkv, D, kc.stride(0), kc.stride(1),
                                              kc.stride(2), min(kc.shape[2], cos.shape[0]), _lib.status_word(qkv.device).data_ptr(),
                                              _lib.DTYPE_CODE[qkv.dtype], _lib.stream_ptr(qkv.device)))
        return q

    def swiglu(self, gu):
        from .. import _lib
        M, f2 = gu.shape
        gu = gu.contiguous()
        out = torch.empty(M, f2 // 2, dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.load().bi_swiglu(gu.data_ptr(), out.data_ptr(), M, f2 // 2, _lib.DTYPE_CODE[gu.dtype],
                                         _lib.stream_ptr(gu.device)))
        return out

    fused_rope = True       # the fold of the qkv projection can rotate and append itself (bi_matmul_rope / bi_qmm_rope)

    def linear_rope(self, x, w, quant, cos, sin, pos0, B, T, hq, hkv, D, kc, vc):
        """rope_append(linear(x, w)) in the matmul's own two launches: returns the rotated q [B, hq, T, D]."""
        q = torch.empty(B, hq, T, D, dtype=x.dtype, device=x.device)
        rope = (cos.data_ptr(), sin.data_ptr(), pos0.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, T, hq, hkv, D,
                kc.stride(0), kc.stride(1), kc.stride(2), min(kc.shape[2], cos.shape[0]))
        if quant is None:
            K.batch_invariant_matmul(x, w.T, rope=rope)
        else:
            p, s, b = w
            K.batch_invariant_quantized_matmul(x, p, s, b, group_size=quant[1], bits=quant[0], rope=rope)
        return q

    fused_wait = True       # the kernels can wait for a peer gather themselves (the *_awaiting entry points)
    fused_push = True       # the matmuls' fold and decode attention's split merge can be the gather (the *_push entry points)

    def add_rms_norm(self, x, delta, w, eps, awaiting=None):
        from .. import _lib
        x, delta = x.contiguous(), delta.contiguous()
        rows, D = x.shape
        s, out = torch.empty_like(x), torch.empty_like(x)
        args = (x.data_ptr(), delta.data_ptr(), w.data_ptr(), s.data_ptr(), out.data_ptr(), rows, D, float(eps),
                _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(x.device))
        if awaiting is None:
            _lib.check(_lib.load().bi_add_rms_norm(*args))
        else:
            _lib.check(_lib.load().bi_add_rms_norm_awaiting(*args, *awaiting, _lib.status_word(x.device).data_ptr()))
        return s, out

    def linear(self, x, w, awaiting=None, push=None):       # x[M, K] @ W[N, K]^T
        return K.batch_invariant_matmul(x, w.T, awaiting=awaiting, push=push)

    def qlinear(self, x, packed, group_size, bits, awaiting=None, push=None):
        p, s, b = packed
        return K.batch_invariant_quantized_matmul(x, p, s, b, group_size=group_size, bits=bits, awaiting=awaiting, push=push)

    def rms_norm(self, x, w, eps):
        return K.batch_invariant_rms_norm(x, w, eps)

    def prefill_attention(self, q, k, v, scale):
        return K.batch_invariant_prefill_attention(q, k, v, scale=scale, causal=True)

    def decode_attention(self, q, k, v, scale, kv_lens=None, push=None):
        return K.batch_invariant_decode_attention(q, k, v, scale=scale, kv_lens=kv_lens, push=push)


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=7).digest(), "little")


def quantize_rows(W: torch.Tensor, group_size: int, bits: int):
    """Affine per-group quantization of W[N, K] on its own device: scale = (max - min)/(2^bits - 1),
    bias = min, code = round((w - bias)/scale) clipped, codes packed low to high in 32-bit words.
    Row-wise, so quantizing a row shard equals the shard of the quantized matrix."""
    N, Kd = W.shape
    dt = W.dtype
    g = W.float().reshape(N, Kd // group_size, group_size)
    lo, hi = g.min(-1).values, g.max(-1).values
    levels = float((1 << bits) - 1)
    scale = ((hi - lo) / levels).clamp_min(1e-8).to(dt)
    bias = lo.to(dt)
    codes = torch.round((g - bias.float()[..., None]) / scale.float()[..., None]).clamp_(0, levels).to(torch.int64)
    per = 32 // bits
    shifts = torch.arange(per, device=W.device, dtype=torch.int64) * bits
    words = (codes.reshape(N, Kd // per, per) << shifts).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words.contiguous(), scale.contiguous(), bias.contiguous()


class ShardedDecoder:
    def __init__(self, cfg: DecoderConfig, *, rank: int = 0, world: int = 1, device="cuda", dtype=torch.bfloat16,
                 quant: tuple[int, int] | None = None, seed: int = 0, group=None, backend=None,
                 max_batch: int = 64, max_len: int = 640):
        if cfg.n_kv_heads % world or cfg.n_heads % world or cfg.ffn % world or cfg.d_model % world or cfg.vocab % world:
            raise ValueError(f"world={world} must divide kv heads, heads, ffn, d_model and vocab")
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        self.dev, self.dt, self.quant, self.seed = torch.device(device), dtype, quant, seed
        self.ops = backend or KernelBackend()
        self.hq, self.hkv = cfg.n_heads // world, cfg.n_kv_heads // world
        D = cfg.head_dim
        self.layers = []
        for li in range(cfg.n_layers):
            wq = self._rows(f"l{li}.wq", cfg.n_heads * D, cfg.d_model, self.hq * D)
            wk = self._rows(f"l{li}.wk", cfg.n_kv_heads * D, cfg.d_model, self.hkv * D)
            wv = self._rows(f"l{li}.wv", cfg.n_kv_heads * D, cfg.d_model, self.hkv * D)
            gate = self._rows(f"l{li}.gate", cfg.ffn, cfg.d_model, cfg.ffn // world)
            up = self._rows(f"l{li}.up", cfg.ffn, cfg.d_model, cfg.ffn // world)
            self.layers.append(dict(
                qkv=self._pack(torch.cat([wq, wk, wv], 0)),
                # the output projection is kept whole on every rank: at decode sizes streaming all of its
                # rows costs less than a sharded product plus the all-gather that would have to follow it
                o=self._pack(self._full(f"l{li}.wo", cfg.d_model, cfg.n_heads * D)),
                gu=self._pack(torch.cat([gate, up], 0)),
                down=self._pack(self._rows(f"l{li}.down", cfg.d_model, cfg.ffn, cfg.d_model // world)),
                n1=self._norm(f"l{li}.n1"), n2=self._norm(f"l{li}.n2")))
            del wq, wk, wv, gate, up
        self.embed = self._full(f"embed", cfg.vocab, cfg.d_model)
        self.head = self._pack(self._rows("lm_head", cfg.vocab, cfg.d_model, cfg.vocab // world))
        self.nf = self._norm("final_norm")
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = torch.arange(max_len, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cat([ang.cos(), ang.cos()], -1).float().to(self.dev)     # [max_len, D]
        self.sin = torch.cat([ang.sin(), ang.sin()], -1).float().to(self.dev)
        self.max_batch, self.max_len = max_batch, max_len
        self.kc = [torch.zeros(max_batch, self.hkv, max_len, D, dtype=dtype, device=self.dev) for _ in range(cfg.n_layers)]
        self.vc = [torch.zeros(max_batch, self.hkv, max_len, D, dtype=dtype, device=self.dev) for _ in range(cfg.n_layers)]
        self.block_hook = None          # callable(layer_index, hidden[B, T, d]) -> None, for per-block hashing
        self._pg = None                 # peer-memory all-gather, created on first use (world > 1, CUDA)

    # ---- weights: every tensor is drawn whole from its own seed, then sliced, so shards of any R agree
    def _gen(self, name):
        g = torch.Generator(device=self.dev)
        g.manual_seed(_tensor_seed(self.seed, name))
        return g

    def _full(self, name, n, k):
        return (torch.randn(n, k, generator=self._gen(name), device=self.dev, dtype=torch.float32) * self.cfg.init_std).to(self.dt)

    def _rows(self, name, n, k, rows_per_rank):
        return self._full(name, n, k)[self.rank * rows_per_rank:(self.rank + 1) * rows_per_rank].contiguous()

    def _norm(self, name):
        return (1.0 + 0.1 * torch.randn(self.cfg.d_model, generator=self._gen(name), device=self.dev, dtype=torch.float32)).to(self.dt)

    def _pack(self, w):
        if self.quant is None:
            return w
        bits, gs = self.quant
        return quantize_rows(w, gs, bits)

    def _add_norm(self, x, delta, w, awaiting=None):
        if awaiting is None:
            return self.ops.add_rms_norm(x, delta, w, self.cfg.eps)
        return self.ops.add_rms_norm(x, delta, w, self.cfg.eps, awaiting=awaiting)

    def _lin(self, x, w, awaiting=None):
        kw = {} if awaiting is None else {"awaiting": awaiting}
        if self.quant is None:
            return self.ops.linear(x, w, **kw)
        return self.ops.qlinear(x, w, self.quant[1], self.quant[0], **kw)

    # ---- collectives: join feature slices [M, F/R] -> [M, F], rank-major (the unsharded order)
    def _gather(self, local, defer=False):
        """Join this rank's feature slice with the others'. defer=True returns (gathered, awaiting): when the
        peer gather is in use and the backend's kernels can wait themselves, the gather kernel does not wait for
        the peers and `awaiting` must be handed to the kernel that reads the result; else `awaiting` is None."""
        if self.world == 1:
            return (local, None) if defer else local
        M, f = local.shape
        local = local.contiguous()
        pg = self._push_gather()
        if pg is not None and pg.fits(M, f * local.element_size()):
            if defer and self._fused_wait():
                return pg.gather(local, wait=False), pg.awaiting()
            out = pg.gather(local)                       # one launch, result already [M, R*f]
            return (out, None) if defer else out
        if defer:
            return self._gather(local), None
        import torch.distributed as dist
        buf = torch.empty(self.world * M, f, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(buf, local, group=self.group)
        return buf.view(self.world, M, f).permute(1, 0, 2).reshape(M, self.world * f)

    def _fused_wait(self) -> bool:
        """Whether the kernels that read a gathered activation wait for it themselves (BI_FUSED_WAIT=0 keeps the
        wait in the gather kernel)."""
        return (getattr(self.ops, "fused_wait", False) and self.dt != torch.float32
                and os.environ.get("BI_FUSED_WAIT", "1") != "0")

    def _qkv(self, h, w, pos0, B, T, kc, vc):
        """The qkv projection, rotary embedding and cache append of a block: rotated q [B, hq, T, D]. With a weight
        on the tensor-core path and decode-sized partials the fold of the projection does all of it
        (BI_FUSED_ROPE=0 keeps the separate kernel)."""
        D = self.cfg.head_dim
        M, Kdim = h.shape
        n = (w[0] if self.quant is not None else w).shape[0]
        fused = (getattr(self.ops, "fused_rope", False) and self.dt != torch.float32
                 and os.environ.get("BI_FUSED_ROPE", "1") != "0"
                 and Kdim % (64 if self.quant is not None else 8) == 0
                 and ((Kdim + 255) // 256) * M * n * 4 <= PUSH_PARTIALS_MAX and vc.stride() == kc.stride()
                 and 256 % D == 0)
        if fused:
            return self.ops.linear_rope(h, w, self.quant, self.cos, self.sin, pos0, B, T, self.hq, self.hkv, D, kc, vc)
        return self.ops.rope_append(self._lin(h, w), self.cos, self.sin, pos0, B, T, self.hq, self.hkv, D, kc, vc)

    def _fused_push(self) -> bool:
        """Whether the kernel that finishes a sharded op's output pushes it to the peers itself (BI_FUSED_PUSH=0
        keeps the separate gather kernel)."""
        return (getattr(self.ops, "fused_push", False) and self.dt != torch.float32
                and os.environ.get("BI_FUSED_PUSH", "1") != "0")

    def _sink(self, rows, cols, defer):
        """(push arguments, local destination, awaiting) of the next peer gather when a kernel can be that gather
        for a [rows, cols] slice, else None."""
        if self.world == 1 or not self._fused_push():
            return None
        pg = self._push_gather()
        if pg is None or not pg.fits(rows, cols * torch.empty(0, dtype=self.dt).element_size()):
            return None
        wait = not (defer and self._fused_wait())
        push, view = pg.sink(rows, cols, self.dt, wait=wait)
        return push, view, (None if wait else pg.awaiting())

    def _lin_gather(self, x, w, awaiting=None, defer=False):
        """_gather(_lin(x, w)). With the peer gather and a weight on the tensor-core path the fold kernel of the
        matmul stores the product into every rank's gathered activation: no local slice, no gather launch."""
        M, Kdim = x.shape
        n = (w[0] if self.quant is not None else w).shape[0]
        groups = (Kdim + 255) // 256
        tc = Kdim % (64 if self.quant is not None else 8) == 0 and groups * M * n * 4 <= PUSH_PARTIALS_MAX
        sk = self._sink(M, n, defer) if tc else None
        if sk is None:
            out = self._gather(self._lin(x, w, awaiting), defer=defer)
            return out
        push, view, aw = sk
        kw = {"push": push}
        if awaiting is not None:
            kw["awaiting"] = awaiting
        if self.quant is None:
            self.ops.linear(x, w, **kw)
        else:
            self.ops.qlinear(x, w, self.quant[1], self.quant[0], **kw)
        return (view, aw) if defer else view

    def _attend_gather(self, q, kk, vv, scale, kv_lens=None):
        """Decode attention of this rank's heads, gathered over the ranks: ([B, hq * world * D], awaiting). With the
        peer gather the split merge stores straight into every rank's gathered activation."""
        B, D = q.shape[0], q.shape[3]
        sk = self._sink(B, self.hq * D, True)
        if sk is None:
            a = self.ops.decode_attention(q, kk, vv, scale, kv_lens=kv_lens)
            return self._gather(a.transpose(1, 2).reshape(B, self.hq * D), defer=True)
        push, view, aw = sk
        self.ops.decode_attention(q, kk, vv, scale, kv_lens=kv_lens, push=push)
        return view, aw

    def _gated(self, gu):
        """SwiGLU of this rank's gate/up slice, gathered over the ranks: [M, 2F/R] -> ([M, F], awaiting). With
        the peer gather the gate is computed inside the gather kernel."""
        if self.world > 1:
            M, f2 = gu.shape
            pg = self._push_gather()
            if pg is not None and gu.is_contiguous() and pg.fits(M, (f2 // 2) * gu.element_size()):
                if self._fused_wait():
                    return pg.gather_swiglu(gu, wait=False), pg.awaiting()
                return pg.gather_swiglu(gu), None
        return self._gather(self.ops.swiglu(gu)), None

    def _push_gather(self):
        """The peer-memory all-gather (CUDA ranks of one node). BI_GATHER=nccl keeps the library collective,
        BI_GATHER=push asks for the peer gather at any world size; unset, it is used at the world sizes it has
        been run at on hardware (PUSH_TESTED_WORLDS) and NCCL elsewhere."""
        if self._pg is None and self.dev.type == "cuda":
            mode = os.environ.get("BI_GATHER", "")
            if mode == "nccl" or (mode != "push" and self.world not in PUSH_TESTED_WORLDS):
                return None
            if getattr(self, "_pg_unavailable", False):
                return None
            from .peer import PeerUnavailable, PushGather
            es = torch.empty(0, dtype=self.dt).element_size()
            widest = max(self.cfg.vocab, self.cfg.ffn, self.cfg.d_model, self.hq * self.world * self.cfg.head_dim)
            try:
                self._pg = PushGather(self.group, self.rank, self.world, self.dev, self.max_batch * widest * es)
            except PeerUnavailable as e:      # raised on all ranks together: all of them take the library collective
                if mode == "push":
                    raise
                self._pg_unavailable = True
                if self.rank == 0:
                    print(f"peer-memory gather unavailable, using NCCL all-gather: {e}", file=sys.stderr)
                return None
        return self._pg

    def check_capacity(self, batch: int, end: int) -> None:
        """Raise before anything is launched if `batch` sequences of `end` tokens do not fit the KV cache and
        the rotary tables (the kernels would otherwise be asked to write past them)."""
        if batch > self.max_batch:
            raise ValueError(f"batch {batch} exceeds the cache's max_batch={self.max_batch}")
        if end > self.max_len:
            raise ValueError(f"position {end} exceeds the cache's max_len={self.max_len}")

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, start: int) -> torch.Tensor:
        """tokens[B, T] continue every sequence at position `start`; returns logits [B, vocab] of the
        last position. T > 1 is a prefill (causal over cache + new keys), T == 1 a decode step."""
        cfg, D = self.cfg, self.cfg.head_dim
        B, T = tokens.shape
        M = B * T
        end = start + T
        self.check_capacity(B, end)
        pos0 = torch.tensor([start], dtype=torch.long, device=self.dev)
        x = self.embed[tokens.reshape(-1)]                                     # [M, d]
        scale = 1.0 / math.sqrt(D)
        h = self.ops.rms_norm(x, self.layers[0]["n1"], cfg.eps)
        for li, L in enumerate(self.layers):
            q = self._qkv(h, L["qkv"], pos0, B, T, self.kc[li], self.vc[li])
            kk, vv = self.kc[li][:B, :, :end], self.vc[li][:B, :, :end]
            if T == 1:
                a, aw = self._attend_gather(q, kk, vv, scale)
            else:
                a = self.ops.prefill_attention(q, kk, vv, scale)
                a, aw = self._gather(a.transpose(1, 2).reshape(M, self.hq * D), defer=True)
            x, h = self.ops.add_rms_norm(x, self._lin(a, L["o"], aw), L["n2"], cfg.eps)
            act, aw = self._gated(self._lin(h, L["gu"]))
            if li + 1 < len(self.layers):       # the add of this block and the first norm of the next, one launch
                delta, aw = self._lin_gather(act, L["down"], aw, defer=True)
                x, h = self._add_norm(x, delta, self.layers[li + 1]["n1"], aw)
            else:
                x = x + self._lin_gather(act, L["down"], aw)
            if self.block_hook is not None:
                self.block_hook(li, x.reshape(B, T, -1))
        last = x.reshape(B, T, -1)[:, -1]
        h = self.ops.rms_norm(last.contiguous(), self.nf, cfg.eps)
        return self._gather(self._lin(h, self.head))


class GraphedDecoder:
    """Greedy decoding with the whole decode step captured once in a CUDA graph.

    Everything that changes from step to step lives on the device -- the position, the per-sequence
    key counts, the token buffer -- so one captured step is replayed for every token: the RoPE / cache
    append kernel reads the position from device memory, attention runs over the
    cache capacity with ``kv_lens``, and the argmax feeds the next step's token buffer. The kernels see
    exactly the calls an eager step makes, so logits are bit-identical to ``ShardedDecoder.forward``.
    """

    def __init__(self, model: ShardedDecoder, batch: int):
        self.m, self.B = model, batch
        dev = model.dev
        self.tokens = torch.zeros(batch, 1, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.lens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.logits = None
        self.graph = None
        self.position = 0                # host mirror of `pos`: every step is checked against the cache before it is launched
        model.check_capacity(batch, 0)

    @torch.no_grad()
    def _step(self):
        m, cfg, B, D = self.m, self.m.cfg, self.B, self.m.cfg.head_dim
        scale = 1.0 / math.sqrt(D)
        x = m.embed[self.tokens.reshape(-1)]
        h = m.ops.rms_norm(x, m.layers[0]["n1"], cfg.eps)
        for li, L in enumerate(m.layers):
            q = m._qkv(h, L["qkv"], self.pos, B, 1, m.kc[li], m.vc[li])
            a, aw = m._attend_gather(q, m.kc[li][:B], m.vc[li][:B], scale, kv_lens=self.lens)
            x, h = m.ops.add_rms_norm(x, m._lin(a, L["o"], aw), L["n2"], cfg.eps)
            act, aw = m._gated(m._lin(h, L["gu"]))
            delta, aw = m._lin_gather(act, L["down"], aw, defer=True)
            nxt = m.layers[li + 1]["n1"] if li + 1 < len(m.layers) else m.nf
            x, h = m._add_norm(x, delta, nxt, aw)
        logits = m._gather(m._lin(h, m.head))
        self.tokens.copy_(logits.argmax(-1, keepdim=True))
        self.pos.add_(1)
        self.lens.add_(1)
        return logits

    def start(self, first_tokens: torch.Tensor, position: int):
        """Continue from `position` (the prompt length) with `first_tokens` [B] as the next input."""
        self.m.check_capacity(self.B, position + 1)
        self.tokens.copy_(first_tokens.reshape(self.B, 1))
        self.pos.fill_(position)
        self.lens.fill_(position + 1)
        self.position = position

    def capture(self):
        """Run one eager step (first-call set-up happens outside capture), rewind, then capture."""
        self.m.check_capacity(self.B, self.position + 1)
        saved = (self.tokens.clone(), self.pos.clone(), self.lens.clone())
        pg = self.m._push_gather() if self.m.world > 1 else None
        before = pg.calls if pg is not None else 0
        self._step()
        torch.cuda.synchronize(self.m.dev)
        if pg is not None:
            pg.set_cycle(pg.calls - before)     # the captured step's gathers repeat back to back
        for dst, src in zip((self.tokens, self.pos, self.lens), saved):
            dst.copy_(src)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._step()
        for dst, src in zip((self.tokens, self.pos, self.lens), saved):
            dst.copy_(src)

    def step(self):
        """Advance every sequence by one token; returns the (static) logits tensor of this step."""
        self.m.check_capacity(self.B, self.position + 1)
        self.position += 1
        if self.graph is None:
            self.logits = self._step()
        else:
            self.graph.replay()
        return self.logits


@torch.no_grad()
def greedy_generate(model: ShardedDecoder, prompts: torch.Tensor, steps: int):
    """Prefill `prompts` [B, P], then `steps` greedy tokens. Returns (tokens [B, steps], last logits)."""
    B, P = prompts.shape
    logits = model.forward(prompts, 0)
    out = []
    for s in range(steps):
        nxt = logits.argmax(-1)
        out.append(nxt)
        if s + 1 < steps:
            logits = model.forward(nxt[:, None], P + s)
    if model.dev.type == "cuda":
        from .. import _lib
        _lib.check_device_status(model.dev)       # a bounded wait that ran out (a gather, a matmul) must not pass silently
    return torch.stack(out, 1), logits
