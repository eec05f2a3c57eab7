"""Host-side sequencing of one pre-LayerNorm encoder block on the C-ABI kernels — the fused form of the node run
the reference's passes produce for a ViT block:

    LayerNorm -> MatMul(Wqkv)+fusedBias -> Reshape/Transpose/Gather (head split) -> Transpose(K) -> MatMul(Q,K^T)
    -> Binary Mul(scale) -> Softmax -> MatMul(P,V) -> Transpose/Reshape (head merge) -> MatMul(Wo)+fusedBias
    -> Add(residual) -> LayerNorm -> MatMul(W1)+fusedBias -> Div/Erf/Add/FusedPointwise (GELU) -> MatMul(W2)+fusedBias
    -> Add(residual)

becomes 7 launches: LN, GEMM(+bias), attention (head split/merge absorbed as strides of the packed qkv buffer),
GEMM(+bias+residual), LN, GEMM(+bias+GELU), GEMM(+bias+residual). The C++ CudaSegment issues the same sequence
after pattern matching; this module exists so tests and the benchmark can drive it without the C++ engine.
"""
from __future__ import annotations

import torch

from . import capi


class EncoderLayer:
    def __init__(self, ctx, weights, heads, dtype=torch.float16, eps=1e-6, device="cuda"):
        """weights: dict of fp32 numpy arrays ln1_g ln1_b wqkv bqkv wo bo ln2_g ln2_b w1 b1 w2 b2; matrices [K,N]."""
        self.ctx, self.H, self.dtype, self.eps = ctx, heads, dtype, eps
        mats = ("wqkv", "wo", "w1", "w2")
        self.w = {}
        for k, v in weights.items():
            t = torch.from_numpy(v).to(device)
            self.w[k] = t.to(dtype).contiguous() if k in mats else t.float().contiguous()
        self.d = self.w["wo"].shape[0]
        self.dmlp = self.w["w1"].shape[1]
        self._buf = {}
        self.cfg = {"qkv": -1, "proj": -1, "fc1": -1, "fc2": -1}  # tensor-core GEMM configuration per GEMM (-1: built-in)

    def _buffers(self, B, T, device):
        key = (B, T)
        if key not in self._buf:
            d, dm, dt = self.d, self.dmlp, self.dtype
            mk = lambda *s: torch.empty(*s, dtype=dt, device=device)  # noqa: E731
            self._buf[key] = dict(h=mk(B * T, d), qkv=mk(B, T, 3, self.H, d // self.H), att=mk(B, T, self.H, d // self.H), x1=mk(B * T, d),
                                  f=mk(B * T, dm))
        return self._buf[key]

    def forward(self, x, out=None):
        """x [B,T,d] in the layer's storage dtype, contiguous. Returns [B,T,d]."""
        c, w = self.ctx, self.w
        B, T, d = x.shape
        H, D = self.H, d // self.H
        buf = self._buffers(B, T, x.device)
        x2 = x.view(B * T, d)
        y = out if out is not None else torch.empty_like(x)
        c.layernorm(x2, w["ln1_g"], w["ln1_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["wqkv"], buf["qkv"].view(B * T, 3 * d), bias=w["bqkv"], config=self.cfg["qkv"])
        qkv = buf["qkv"]                                  # [B,T,3,H,D]
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))   # [B,H,T,D] strided views, no copy
        o = buf["att"].permute(0, 2, 1, 3)                # attention writes straight into the merged [B,T,H*D] layout
        c.attn_prefill(q, k, v, o, scale=1.0 / (D ** 0.5))
        c.gemm(buf["att"].view(B * T, d), w["wo"], buf["x1"], bias=w["bo"], residual=x2, config=self.cfg["proj"])
        c.layernorm(buf["x1"], w["ln2_g"], w["ln2_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["w1"], buf["f"], bias=w["b1"], epilogue=capi.EPI_BIAS | capi.EPI_GELU_ERF, config=self.cfg["fc1"])
        c.gemm(buf["f"], w["w2"], y.view(B * T, d), bias=w["b2"], residual=buf["x1"], config=self.cfg["fc2"])
        return y

    def tune(self, x, iters=10, table=None):
        """Per-shape choice of the GEMM configuration by measurement, as CudaSegment::tuneGemms does at plan time
        (Hint::Tuning). `table` (dict) carries choices between layers of the same shape so each shape is timed once."""
        c, w = self.ctx, self.w
        B, T, d = x.shape
        buf = self._buffers(B, T, x.device)
        x2, y = x.view(B * T, d), torch.empty_like(x).view(B * T, d)
        gemms = {
            "qkv": lambda cfg: c.gemm(buf["h"], w["wqkv"], buf["qkv"].view(B * T, 3 * d), bias=w["bqkv"], config=cfg),
            "proj": lambda cfg: c.gemm(buf["att"].view(B * T, d), w["wo"], buf["x1"], bias=w["bo"], residual=x2, config=cfg),
            "fc1": lambda cfg: c.gemm(buf["h"], w["w1"], buf["f"], bias=w["b1"], epilogue=capi.EPI_BIAS | capi.EPI_GELU_ERF, config=cfg),
            "fc2": lambda cfg: c.gemm(buf["f"], w["w2"], y, bias=w["b2"], residual=buf["x1"], config=cfg),
        }
        table = {} if table is None else table
        for name, fn in gemms.items():
            key = (name, B * T, d, self.dmlp)
            if key not in table:
                best, best_ms = -1, float("inf")
                for cfg in range(-1, c.gemm_config_count()):
                    try:
                        fn(cfg), fn(cfg)
                    except RuntimeError:
                        continue  # a configuration this shape cannot run
                    # time on the device: `iters` launches replayed as one CUDA graph (eager launches from Python are
                    # host-bound at these kernel lengths and would rank the configurations by noise)
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for _ in range(iters):
                            fn(cfg)
                    g.replay()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g.replay()
                    g.replay()
                    e1.record()
                    e1.synchronize()
                    ms = e0.elapsed_time(e1)
                    if ms < best_ms * 0.97:
                        best, best_ms = cfg, ms
                table[key] = best
            self.cfg[name] = table[key]
        return table

    LAUNCHES_PER_FORWARD = 7

    def capture(self, x, out):
        """Records forward(x, out) into a CUDA graph (the launch list of a segment, replayable with .replay()).
        One eager call must have run before so that every kernel's one-time set-up is done."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward(x, out=out)
        return g

    # ---- head-sharded form for a single long sequence (batch 1 cannot be sharded by batch) ---------------------
    def shard_heads(self, rank, world):
        """Keeps only this rank's heads of the QKV projection (columns of Wqkv / entries of bqkv). Attention then runs
        on H/world heads per rank; the attention output is all-gathered before the replicated out-projection + MLP."""
        from .sharding import qkv_head_slice
        assert self.H % world == 0
        self.w["wqkv_local"], self.w["bqkv_local"] = qkv_head_slice(self.w["wqkv"], self.w["bqkv"], self.H, rank, world)
        self.rank, self.world, self.Hl = rank, world, self.H // world

    def forward_head_sharded(self, x, group=None, out=None):
        """x [1,T,d] replicated on every rank. One NCCL all-gather per layer, at the attention-output boundary."""
        import torch.distributed as dist
        c, w = self.ctx, self.w
        B, T, d = x.shape
        assert B == 1
        H, Hl, D, world = self.H, self.Hl, d // self.H, self.world
        dl = Hl * D
        buf = self._buffers(B, T, x.device)
        key = ("hs", T)
        if key not in self._buf:
            mk = lambda *s_: torch.empty(*s_, dtype=self.dtype, device=x.device)  # noqa: E731
            self._buf[key] = dict(qkv=mk(T, 3, Hl, D), att=mk(T, Hl, D), gathered=mk(world, T, dl))
        hs = self._buf[key]
        x2 = x.view(T, d)
        y = out if out is not None else torch.empty_like(x)
        c.layernorm(x2, w["ln1_g"], w["ln1_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["wqkv_local"], hs["qkv"].view(T, 3 * dl), bias=w["bqkv_local"])
        q, k, v = (hs["qkv"][:, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))      # [1,Hl,T,D] views
        c.attn_prefill(q, k, v, hs["att"].permute(1, 0, 2).unsqueeze(0), scale=1.0 / (D ** 0.5))
        dist.all_gather_into_tensor(hs["gathered"].view(world * T, dl), hs["att"].view(T, dl), group=group)
        # [world,T,dl] -> [T, world*dl]: heads are contiguous per rank, so this restores the merged-head layout
        att_full = buf["att"].view(T, d)
        c.strided_copy(hs["gathered"], att_full, [T, world, dl], [dl, T * dl, 1])
        c.gemm(att_full, w["wo"], buf["x1"], bias=w["bo"], residual=x2)
        c.layernorm(buf["x1"], w["ln2_g"], w["ln2_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["w1"], buf["f"], bias=w["b1"], epilogue=capi.EPI_BIAS | capi.EPI_GELU_ERF)
        c.gemm(buf["f"], w["w2"], y.view(T, d), bias=w["b2"], residual=buf["x1"])
        return y

    def forward_head_sharded_fused(self, x, gather, out=None):
        """Like forward_head_sharded, without a collective: the attention kernel stores its output tiles straight into every
        rank's gather buffer (sharding.PeerGather) and publishes a flag; the out-projection reads this rank's buffer after a
        bounded device-side wait on the flags. Only this library's kernels run, so the whole stack captures into one CUDA graph."""
        c, w = self.ctx, self.w
        B, T, d = x.shape
        assert B == 1 and gather.rows == T and gather.width == d
        Hl, D = self.Hl, d // self.H
        dl = Hl * D
        buf = self._buffers(B, T, x.device)
        key = ("hsf", T)
        if key not in self._buf:
            self._buf[key] = dict(qkv=torch.empty(T, 3, Hl, D, dtype=self.dtype, device=x.device))
        hs = self._buf[key]
        x2 = x.view(T, d)
        y = out if out is not None else torch.empty_like(x)
        c.layernorm(x2, w["ln1_g"], w["ln1_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["wqkv_local"], hs["qkv"].view(T, 3 * dl), bias=w["bqkv_local"])
        q, k, v = (hs["qkv"][:, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))      # [1,Hl,T,D] views
        kbuf = gather.next_buffer()
        # output element (head h, row t, :) of this rank lands at [t, (rank*Hl + h)*D : ...] of every rank's [T, d] buffer
        c.attn_prefill_fanout(q, k, v, gather.dests(kbuf, self.rank * dl), gather.flags(), gather.state, (T * d, D, d), scale=1.0 / (D ** 0.5),
                              mcast=gather.mcast(kbuf, self.rank * dl))
        # the out-projection's own producer warp waits for the ranks' flags (no wait kernel between the two launches)
        c.gemm(gather.buffers[kbuf], w["wo"], buf["x1"], bias=w["bo"], residual=x2, gate=gather.gate())
        c.layernorm(buf["x1"], w["ln2_g"], w["ln2_b"], buf["h"], self.eps)
        c.gemm(buf["h"], w["w1"], buf["f"], bias=w["b1"], epilogue=capi.EPI_BIAS | capi.EPI_GELU_ERF)
        c.gemm(buf["f"], w["w2"], y.view(T, d), bias=w["b2"], residual=buf["x1"])
        return y

    def forward_token_sharded(self, x_loc, rows, T, gather_h, gather_att, out=None):
        """One block with EVERYTHING sharded and no collective call: this rank holds rows [rows[0], rows[1]) of the residual
        stream (x_loc [Tl, d]) and heads [rank*Hl, (rank+1)*Hl). LayerNorm 1 stores its normalised rows into every rank's
        `gather_h` buffer (each rank's QKV projection needs all tokens for its own heads); the attention kernel stores its
        heads' output for all tokens into every rank's `gather_att` buffer; out-projection, LayerNorm 2 and the MLP then run on
        this rank's rows only. Returns the rank's rows of the block output."""
        c, w = self.ctx, self.w
        lo, hi = rows
        Tl, d = x_loc.shape
        assert Tl == hi - lo
        Hl, D, dm = self.Hl, d // self.H, self.dmlp
        dl = Hl * D
        key = ("ts", T, Tl)
        if key not in self._buf:
            mk = lambda *s_: torch.empty(*s_, dtype=self.dtype, device=x_loc.device)  # noqa: E731
            self._buf[key] = dict(qkv=mk(T, 3, Hl, D), x1=mk(Tl, d), h=mk(Tl, d), f=mk(Tl, dm))
        b = self._buf[key]
        y = out if out is not None else torch.empty_like(x_loc)
        kh = gather_h.next_buffer()
        c.layernorm_fanout(x_loc, w["ln1_g"], w["ln1_b"], gather_h.dests(kh, lo * d), gather_h.flags(), gather_h.state, self.eps,
                           mcast=gather_h.mcast(kh, lo * d))
        c.gemm(gather_h.buffers[kh], w["wqkv_local"], b["qkv"].view(T, 3 * dl), bias=w["bqkv_local"], gate=gather_h.gate())
        q, k, v = (b["qkv"][:, i].permute(1, 0, 2).unsqueeze(0) for i in range(3))
        ka = gather_att.next_buffer()
        c.attn_prefill_fanout(q, k, v, gather_att.dests(ka, self.rank * dl), gather_att.flags(), gather_att.state, (T * d, D, d),
                              scale=1.0 / (D ** 0.5), mcast=gather_att.mcast(ka, self.rank * dl))
        c.gemm(gather_att.buffers[ka][lo:hi], w["wo"], b["x1"], bias=w["bo"], residual=x_loc, gate=gather_att.gate())
        c.layernorm(b["x1"], w["ln2_g"], w["ln2_b"], b["h"], self.eps)
        c.gemm(b["h"], w["w1"], b["f"], bias=w["b1"], epilogue=capi.EPI_BIAS | capi.EPI_GELU_ERF)
        c.gemm(b["f"], w["w2"], y, bias=w["b2"], residual=b["x1"])
        return y

    def flops(self, B, T):
        d, dm, H = self.d, self.dmlp, self.H
        M = B * T
        return 2 * M * d * 3 * d + 4 * B * H * T * T * (d // H) + 2 * M * d * d + 4 * M * d * dm


class EncoderStack:
    """A stack of identical-shape pre-LN blocks with independent weights (the 24-layer encoder of config 3)."""

    def __init__(self, ctx, weights_per_layer, heads, dtype=torch.float16, eps=1e-6):
        self.layers = [EncoderLayer(ctx, w, heads, dtype=dtype, eps=eps) for w in weights_per_layer]
        self._pp = {}

    def _pingpong(self, x):
        key = tuple(x.shape)
        if key not in self._pp:
            self._pp[key] = [torch.empty_like(x), torch.empty_like(x)]
        return self._pp[key]

    def tune(self, x):
        table = {}
        for layer in self.layers:
            layer.tune(x, table=table)
        return table

    def forward(self, x):
        """Ping-pongs between two internal buffers; the caller's input is left untouched."""
        cur, bufs = x, self._pingpong(x)
        for i, layer in enumerate(self.layers):
            cur = layer.forward(cur, out=bufs[i % 2])
        return cur

    def shard_heads(self, rank, world):
        for layer in self.layers:
            layer.shard_heads(rank, world)

    def forward_head_sharded(self, x, group=None):
        cur, bufs = x, self._pingpong(x)
        for i, layer in enumerate(self.layers):
            cur = layer.forward_head_sharded(cur, group=group, out=bufs[i % 2])
        return cur

    def forward_head_sharded_fused(self, x, gather):
        """All layers with the attention output fanned out by the attention kernel (no collective). The two gather buffers
        alternate per layer, so an even number of layers keeps the alternation intact from one forward to the next."""
        assert len(self.layers) % 2 == 0, "an odd layer count would reuse a gather buffer that a slower rank may still read"
        cur, bufs = x, self._pingpong(x)
        for i, layer in enumerate(self.layers):
            cur = layer.forward_head_sharded_fused(cur, gather, out=bufs[i % 2])
        return cur

    def forward_token_sharded(self, x, gather_h, gather_att):
        """x [1,T,d] replicated; returns this rank's rows [Tl, d] of the stack output (sharding.shard_range(T, rank, world)).
        Heads and tokens are both sharded; the two all-gathers per layer are done by the LayerNorm and attention kernels
        themselves over peer memory. Needs shard_heads() first and an even layer count (the gather buffers alternate)."""
        from .sharding import shard_range
        assert len(self.layers) % 2 == 0, "an odd layer count would reuse a gather buffer that a slower rank may still read"
        T, d = x.shape[1], x.shape[2]
        rank, world = self.layers[0].rank, self.layers[0].world
        lo, hi = shard_range(T, rank, world)
        key = ("ts", T, hi - lo)
        if key not in self._pp:
            self._pp[key] = [torch.empty(hi - lo, d, dtype=x.dtype, device=x.device) for _ in range(2)]
        cur = x.view(T, d)[lo:hi]
        for i, layer in enumerate(self.layers):
            cur = layer.forward_token_sharded(cur, (lo, hi), T, gather_h, gather_att, out=self._pp[key][i % 2])
        return cur

    def capture_token_sharded(self, x, gather_h, gather_att):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = self.forward_token_sharded(x, gather_h, gather_att)
        return g, y

    def capture_head_sharded_fused(self, x, gather):
        """CUDA graph of forward_head_sharded_fused; needs one eager call on every rank beforehand."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = self.forward_head_sharded_fused(x, gather)
        return g, y

    def capture(self, x):
        """CUDA graph of forward(x); returns (graph, output tensor). Needs one eager forward beforehand."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = self.forward(x)
        return g, y

    def flops(self, B, T):
        return sum(layer.flops(B, T) for layer in self.layers)
