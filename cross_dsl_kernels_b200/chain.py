"""The Llama-3-8B-shaped decode-layer chain built from the four kernels.

Per layer and decode step (batch of ``tokens`` rows, FP16 activations):

1. residual RMSNorm                     (h, residual) -> (n1, r1)
2. W4A16 QKV projection                 n1 -> qkv   [tokens, (q_heads + 2 kv_heads) * head_dim]
3. RoPE + paged K/V append              q, k, v are column slices of qkv (no copy); returns rotated q
4. residual RMSNorm                     (rotated q as the hidden stream, r1) -> (n2, r2)
5. W4A16 MLP up+gate projection         n2 -> upgate [tokens, 2 * mlp]

The five-kernel chain has no attention between 3 and 4 (it is not one of the
four kernels): the rotated Q -- which has the hidden width -- stands in for the
attention output and keeps the five launches data-dependent.  With
``attention=True`` (single GPU) the two ops that follow the path are inserted:

3b. paged decode attention over the cache step 3 wrote   q_rot -> attn [tokens, hidden]
5b. SwiGLU on the up+gate output                          upgate -> act [tokens, mlp]

Multi-GPU (one process per GPU): the projections are column-sharded and the KV
heads split, rank r owning q heads [r*Hq/g, ...), kv heads [r*Hkv/g, ...) and
the same fraction of the up+gate columns; its QKV shard is laid out
[its Q heads | its K heads | its V heads], i.e. exactly what its RoPE/append
launch consumes, so nothing is exchanged before the append and every rank keeps
its own KV-cache shard.  The rotated Q shards and the up+gate shards have to
reach every rank; two ways are built:

* ``exchange="peer"`` (default): the append kernel and the up+gate projection
  store their shard into the right columns of the full-width matrix in EVERY
  rank's peer-mapped arena from their epilogues (peer.py), and one flag barrier
  per exchange point orders the readers.  No collective, no re-layout kernel.
* ``exchange="nccl"``: all-gather over NCCL (rank-major) and a small kernel that
  re-lays the result row-major -- kept as the comparison arm.

``dependent_launch=True`` launches every kernel of the chain as a programmatic
dependent of its predecessor, so that scheduling, set-up and (for the
projections) the first weight tiles overlap the predecessor's tail.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native
from .ops import fused_residual_rmsnorm, rope_gqa_paged_kv_append
from .quantization import pack_int4
from .w4a16 import w4a16_linear


@dataclass
class ChainConfig:
    tokens: int = 16
    hidden: int = 4096
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    mlp: int = 14336
    context: int = 8192
    page_size: int = 16
    group: int = 128
    theta: float = 10000.0
    eps: float = 1e-6

    @property
    def qkv_cols(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim

    def algorithmic_bytes(self) -> int:
        from . import workloads as wl

        t, h = self.tokens, self.hidden
        return (2 * wl.rmsnorm_bytes(t, h, torch.float16)
                + wl.w4a16_bytes(t, h, self.qkv_cols, self.group)
                + wl.rope_bytes(t, self.q_heads, self.kv_heads, self.head_dim, self.head_dim, torch.float16)
                + wl.w4a16_bytes(t, h, 2 * self.mlp, self.group))


def qkv_shard_rows(cfg: ChainConfig, rank: int, world: int) -> torch.Tensor:
    """Rows of the fused QKV weight ([Q heads | K heads | V heads] x head_dim) that rank ``rank`` owns,
    in the order its shard stores them: its Q heads, then its K heads, then its V heads."""
    d = cfg.head_dim
    hq, hkv = cfg.q_heads // world, cfg.kv_heads // world
    k0, v0 = cfg.q_heads * d, (cfg.q_heads + cfg.kv_heads) * d
    return torch.cat([torch.arange(rank * hq * d, (rank + 1) * hq * d),
                      torch.arange(k0 + rank * hkv * d, k0 + (rank + 1) * hkv * d),
                      torch.arange(v0 + rank * hkv * d, v0 + (rank + 1) * hkv * d)])


def upgate_shard_rows(cfg: ChainConfig, rank: int, world: int, paired: bool = False) -> torch.Tensor:
    """Rows (output columns) of the up+gate weight that rank ``rank`` owns.  Plain: one contiguous block of the
    [up | gate] matrix.  ``paired`` (the layer applies SwiGLU): the rank's block of up columns followed by the same
    block of gate columns, so that the activation of those columns needs nothing from another rank."""
    if paired:
        cols = cfg.mlp // world
        return torch.cat([torch.arange(rank * cols, (rank + 1) * cols), torch.arange(cfg.mlp + rank * cols, cfg.mlp + (rank + 1) * cols)])
    cols = 2 * cfg.mlp // world
    return torch.arange(rank * cols, (rank + 1) * cols)


def unshard_reference(gathered: torch.Tensor) -> torch.Tensor:
    """What :func:`unshard_columns` computes, as a tensor expression (any device)."""
    world, rows, cols = gathered.shape
    return gathered.permute(1, 0, 2).reshape(rows, world * cols)


def _quantised(n: int, k: int, group: int, gen: torch.Generator):
    """Codes uniform in [0, 15], scales uniform in [0.005, 0.02]; drawn on the generator's device."""
    dev = gen.device
    codes = torch.randint(0, 16, (n, k), generator=gen, device=dev, dtype=torch.int8)
    packed = pack_int4(codes - 8)
    scales = (0.005 + 0.015 * torch.rand(n, k // group, generator=gen, device=dev)).half()
    return packed, scales


def unshard_columns(gathered: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """[world, rows, cols] (rank-major all-gather result) -> out[rows, world*cols]."""
    world, rows, cols = gathered.shape
    status = _native.lib().xdk_unshard_columns(gathered.data_ptr(), out.data_ptr(), world, rows, cols,
                                               gathered.element_size(), _native.stream_ptr(gathered.device))
    _native.check(status, "xdk_unshard_columns")
    return out


class DecodeLayerChain:
    """Weights, caches and index tensors of ``layers`` identical-shape layers for one rank."""

    def __init__(self, cfg: ChainConfig = ChainConfig(), *, layers: int = 1, rank: int = 0, world: int = 1,
                 seed: int = 0, device="cuda", group=None, exchange: str = "peer", dependent_launch: bool = False,
                 attention: bool = False):
        if cfg.q_heads % world or cfg.kv_heads % world or (2 * cfg.mlp) % world:
            raise ValueError("heads and MLP columns must divide by the number of ranks")
        if exchange not in ("peer", "nccl"):
            raise ValueError("exchange must be 'peer' or 'nccl'")
        if attention and world > 1 and exchange != "peer":
            raise ValueError("the sharded chain with attention exchanges through peer-mapped stores only")
        self.cfg, self.rank, self.world, self.pg = cfg, rank, world, group
        self.exchange, self.dependent = exchange, bool(dependent_launch)
        self.attention = bool(attention)
        self.device = torch.device(device)
        c = cfg
        # Weights are drawn on the device (Philox, same values on every rank for one seed): drawing
        # 4 x 140 M codes on one host thread per rank would dominate a multi-rank start-up.
        wgen = torch.Generator(device=self.device).manual_seed(seed)
        gen = torch.Generator().manual_seed(seed)
        d = c.head_dim
        hq, hkv = c.q_heads // world, c.kv_heads // world
        self.local_q_heads, self.local_kv_heads = hq, hkv
        self.layers = []
        for _ in range(layers):
            w1 = (1 + 0.1 * torch.randn(c.hidden, generator=gen)).half()
            w2 = (1 + 0.1 * torch.randn(c.hidden, generator=gen)).half()
            qkv_p, qkv_s = _quantised(c.qkv_cols, c.hidden, c.group, wgen)
            up_p, up_s = _quantised(2 * c.mlp, c.hidden, c.group, wgen)
            rows = qkv_shard_rows(c, rank, world).to(self.device)
            up_rows = upgate_shard_rows(c, rank, world, paired=attention and world > 1).to(self.device)
            layer = dict(
                w1=w1.to(self.device), w2=w2.to(self.device),
                qkv_packed=qkv_p[rows].contiguous(), qkv_scales=qkv_s[rows].contiguous(),
                up_packed=up_p[up_rows].contiguous(), up_scales=up_s[up_rows].contiguous())
            if world == 1:  # full (unsharded) weights for checkers; copied to the host only when asked for
                layer["full"] = dict(w1=w1, w2=w2, qkv_packed=qkv_p, qkv_scales=qkv_s, up_packed=up_p, up_scales=up_s)
            self.layers.append(layer)
        pages_per_seq = c.context // c.page_size
        pages = c.tokens * pages_per_seq
        self.positions = torch.randint(0, c.context, (c.tokens,), generator=gen)
        self.sequence_ids = torch.arange(c.tokens)
        self.page_table = torch.randperm(pages, generator=gen).reshape(c.tokens, pages_per_seq)
        inv_freq = c.theta ** (-torch.arange(0, d, 2).float() / d)
        angle = torch.arange(c.context).float()[:, None] * inv_freq[None, :]
        self.cos, self.sin = angle.cos(), angle.sin()
        self.h = torch.randn(c.tokens, c.hidden, generator=gen).half()
        self.res = torch.randn(c.tokens, c.hidden, generator=gen).half()
        self.dev = {k: getattr(self, k).to(self.device) for k in
                    ("positions", "sequence_ids", "page_table", "cos", "sin", "h", "res")}
        shape = (pages, c.page_size, hkv, d)
        self.k_cache = torch.full(shape, -999.0, dtype=torch.float16, device=self.device)
        self.v_cache = torch.full(shape, -999.0, dtype=torch.float16, device=self.device)
        self.arena = None
        if world > 1 and exchange == "peer":
            from .peer import PeerArena

            # two copies of each full-width matrix, used by alternate layers: a rank that runs ahead into the
            # next layer never stores into a matrix a slower rank is still reading
            nbytes = 2 * (c.tokens * c.hidden + c.tokens * 2 * c.mlp) * 2 + 4096
            self.arena = PeerArena(nbytes, group=group, device=self.device)
            # with attention: the attention output (sharded by KV head) and the activation (sharded by MLP column) are
            # what the ranks assemble for one another; without it, rotated Q and the up+gate projection
            self.q_peer = [self.arena.matrix(c.tokens, c.hidden, torch.float16) for _ in range(2)]
            self.up_peer = [self.arena.matrix(c.tokens, c.mlp if attention else 2 * c.mlp, torch.float16) for _ in range(2)]
            self.site_q, self.site_up = self.arena.new_site(), self.arena.new_site()
            self.launches_per_layer = 9 if attention else 7  # the kernels + two flag barriers
        elif world > 1:
            self.q_gather = torch.empty(world, c.tokens, hq * d, dtype=torch.float16, device=self.device)
            self.up_gather = torch.empty(world, c.tokens, 2 * c.mlp // world, dtype=torch.float16, device=self.device)
            self.q_full = torch.empty(c.tokens, c.hidden, dtype=torch.float16, device=self.device)
            self.up_full = torch.empty(c.tokens, 2 * c.mlp, dtype=torch.float16, device=self.device)
            self.launches_per_layer = 7  # five kernels + two re-layout kernels (+ two NCCL all-gathers)
        else:
            self.launches_per_layer = 7 if attention else 5

    def host_weights(self, layer: int = 0) -> dict:
        """CPU copies of one layer's unsharded weights (single-rank chains only; for checkers)."""
        return {k: v.cpu() for k, v in self.layers[layer]["full"].items()}

    def step(self, layer: int = 0, h=None, res=None) -> dict:
        """One layer: returns every intermediate (device tensors)."""
        import torch.distributed as dist

        c, L, dv = self.cfg, self.layers[layer], self.dev
        d, hq, hkv = c.head_dim, self.local_q_heads, self.local_kv_heads
        dep = self.dependent
        peer = self.arena is not None
        h = dv["h"] if h is None else h
        res = dv["res"] if res is None else res
        n1, r1 = fused_residual_rmsnorm(h, res, L["w1"], c.eps, dependent_launch=dep)
        qkv = w4a16_linear(n1, L["qkv_packed"], L["qkv_scales"], None, group_size=c.group, dependent_launch=dep)
        q = qkv[:, : hq * d].view(c.tokens, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(c.tokens, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(c.tokens, hkv, d)
        q_dst = self.q_peer[layer % 2] if peer else None
        sharded_attention = peer and self.attention
        q_rot = rope_gqa_paged_kv_append(q, k, v, dv["cos"], dv["sin"], dv["positions"], dv["page_table"],
                                         dv["sequence_ids"], self.k_cache, self.v_cache, page_size=c.page_size,
                                         rope_dim=d, interleaved=False, kv_layout="NHD", dependent_launch=dep,
                                         q_peer_out=q_dst.out_for(self.rank * hq * d) if peer and not sharded_attention else None)
        if sharded_attention:
            from .ops import paged_decode_attention

            # this rank's heads against its own cache shard; every rank receives the result
            paged_decode_attention(q_rot, self.k_cache, self.v_cache, dv["positions"], dv["page_table"], dv["sequence_ids"],
                                   page_size=c.page_size, context_hint=c.context, dependent_launch=dep,
                                   peer_out=q_dst.out_for(self.rank * hq * d))
            self.arena.barrier(self.site_q, dependent_launch=dep)
            attn = q_dst.local
        elif peer:
            self.arena.barrier(self.site_q, dependent_launch=dep)
            attn = q_dst.local
        elif self.world > 1:
            dist.all_gather_into_tensor(self.q_gather, q_rot.view(c.tokens, hq * d), group=self.pg)
            attn = unshard_columns(self.q_gather, self.q_full)
        elif self.attention:
            from .ops import paged_decode_attention

            attn = paged_decode_attention(q_rot, self.k_cache, self.v_cache, dv["positions"], dv["page_table"], dv["sequence_ids"],
                                          page_size=c.page_size, context_hint=c.context, dependent_launch=dep).view(c.tokens, c.hidden)
        else:
            attn = q_rot.view(c.tokens, c.hidden)
        n2, r2 = fused_residual_rmsnorm(attn, r1, L["w2"], c.eps, dependent_launch=dep)
        if sharded_attention:
            from .ops import swiglu

            act_dst = self.up_peer[layer % 2]
            up = w4a16_linear(n2, L["up_packed"], L["up_scales"], None, group_size=c.group, dependent_launch=dep)  # [up_r | gate_r]
            swiglu(up, dependent_launch=dep, peer_out=act_dst.out_for(self.rank * (c.mlp // self.world)))
            self.arena.barrier(self.site_up, dependent_launch=dep)
            return dict(n1=n1, r1=r1, qkv=qkv, q_rot=q_rot, attn=attn, n2=n2, r2=r2, up=up, up_all=None, act=act_dst.local)
        if peer:
            up_dst = self.up_peer[layer % 2]
            w4a16_linear(n2, L["up_packed"], L["up_scales"], None, group_size=c.group, dependent_launch=dep,
                         peer_out=up_dst.out_for(self.rank * (2 * c.mlp // self.world)))
            self.arena.barrier(self.site_up, dependent_launch=dep)
            up = up_dst.local[:, self.rank * (2 * c.mlp // self.world): (self.rank + 1) * (2 * c.mlp // self.world)]
            up_all = up_dst.local
        else:
            up = w4a16_linear(n2, L["up_packed"], L["up_scales"], None, group_size=c.group, dependent_launch=dep)
            if self.world > 1:
                dist.all_gather_into_tensor(self.up_gather, up, group=self.pg)
                up_all = unshard_columns(self.up_gather, self.up_full)
            else:
                up_all = up
        out = dict(n1=n1, r1=r1, qkv=qkv, q_rot=q_rot, attn=attn, n2=n2, r2=r2, up=up, up_all=up_all)
        if self.attention:
            from .ops import swiglu

            out["act"] = swiglu(up_all, dependent_launch=dep)
        return out

    def run_layers(self):
        """All layers back to back, each feeding the next its (n2, r2)."""
        h = res = None
        out = None
        for i in range(len(self.layers)):
            out = self.step(i, h, res)
            h, res = out["n2"], out["r2"]
        return out
