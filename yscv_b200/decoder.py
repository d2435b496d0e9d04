"""Random-init int4 Llama-shape decoder on top of the C ABI.

The reference has no native decoder: `apps/llm-bench` runs an exported ONNX graph
whose MatMul nodes hit the packed-int4 side-table (apps/llm-bench/src/main.rs:315-593,
crates/yscv-onnx/src/runner/linear.rs:223-278). This module assembles the same
operator sequence (RMSNorm, fused QKV linear, rotate-half RoPE, KV-cache append, GQA
attention, output linear, SwiGLU MLP, fp32 LM head, greedy argmax-last) from the
library's entry points, so the int4 kernels can be measured in the loop they exist
for. Every tensor operation is a call into libyscv_cuda.so; torch supplies device
memory, the stream, the CUDA graph that replays a decode step, and (tensor
parallel) the rendezvous between the ranks and the NCCL all-reduce of the prompt pass.

Tensor parallel layout (tp_size ranks): q/k/v heads, gate and up rows are split
across ranks (column-parallel, no collective); the output and down projections are
split along K (row-parallel) and their fp32 partial sums are summed across the ranks:
by `ncclAllReduce` in the operator chain (prompt pass, batch > 1), and inside the
one-launch decode step by the kernel itself (peer stores into exchange regions the
ranks map through CUDA IPC, sums in rank order), where the LM head is split by rows too.

`kv_int8=True` stores the KV cache as the reference's KvDtype::I8
(crates/yscv-onnx/src/runner/kv_cache.rs:8-90): int8 rows with one f32 scale per token.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import sharding
from .lib import Context, TpComm, YscvCudaError, TP_HANDLE_BYTES


@dataclass(frozen=True)
class DecoderConfig:
    layers: int
    hidden: int
    mlp: int
    n_q: int
    n_kv: int
    head_dim: int
    vocab: int
    eps: float = 1e-5
    rope_theta: float = 10000.0
    group_size: int = 32
    weight_std: float = 0.02


TINYLLAMA_1B = DecoderConfig(22, 2048, 5632, 32, 4, 64, 32000, 1e-5, 10000.0)
LLAMA3_70B = DecoderConfig(80, 8192, 28672, 64, 8, 128, 128256, 1e-5, 500000.0)


class Int4Linear:
    """A packed int4 weight [n][k] resident on the device."""

    def __init__(self, ctx: Context, packed: torch.Tensor, scales: torch.Tensor, n: int, k: int, g: int):
        self.packed, self.scales, self.n, self.k, self.g = packed, scales, n, k, g
        self.handle = ctx.int4_weight_wrap(packed.data_ptr(), scales.data_ptr(), n, k, g)


class Int4Decoder:
    def __init__(self, ctx: Context, cfg: DecoderConfig, batch: int, max_seq: int, stream: torch.cuda.Stream,
                 seed: int = 3, tp_rank: int = 0, tp_size: int = 1, process_group=None,
                 layers: int | None = None, fused_step: bool = True, kv_int8: bool = False,
                 plan_options: dict | None = None):
        assert cfg.n_q % tp_size == 0 and cfg.n_kv % tp_size == 0 and cfg.mlp % (tp_size * cfg.group_size) == 0
        self.ctx, self.cfg, self.batch, self.max_seq, self.stream = ctx, cfg, batch, max_seq, stream
        self.tp_rank, self.tp_size, self.pg = tp_rank, tp_size, process_group
        self.n_layers = layers if layers is not None else cfg.layers
        self.dev = torch.device("cuda", ctx.device)
        self.nq_l, self.nkv_l, self.mlp_l = cfg.n_q // tp_size, cfg.n_kv // tp_size, cfg.mlp // tp_size
        self.seed = seed
        self.full = {}  # unsharded packed weights kept only when asked (parity tests read them back)
        with torch.cuda.stream(stream):
            self._build_weights()
            d, B = cfg.head_dim, batch
            self.kv_int8 = kv_int8
            kv_dtype = torch.int8 if kv_int8 else torch.float32
            self.kcache = [torch.zeros(B, max_seq, self.nkv_l, d, dtype=kv_dtype, device=self.dev) for _ in range(self.n_layers)]
            self.vcache = [torch.zeros(B, max_seq, self.nkv_l, d, dtype=kv_dtype, device=self.dev) for _ in range(self.n_layers)]
            if kv_int8:  # one scale per cached row (token), keys and values apart
                self.kscale = [torch.zeros(B, max_seq, device=self.dev) for _ in range(self.n_layers)]
                self.vscale = [torch.zeros(B, max_seq, device=self.dev) for _ in range(self.n_layers)]
            self.pos = torch.zeros(1, dtype=torch.int32, device=self.dev)
            self.next_tokens = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self._bufs = {}
        self.graph = None
        stream.synchronize()
        # batch 1: the whole single-token step as one persistent kernel per GPU, when the
        # shapes allow it (the library says which do). With tensor parallelism the ranks'
        # kernels exchange their partial sums through exchange regions mapped with CUDA IPC;
        # the handles travel through the process group, and every rank must agree on whether
        # the plan exists.
        self.plan = None
        self.tp_comm = None
        self.lm_row0, self.lm_rows = 0, cfg.vocab
        # batches of 2..8 sequences take the batch form of the same kernel (one GPU, f32 caches)
        if fused_step and (batch == 1 or (batch <= 8 and tp_size == 1 and not kv_int8)):
            try:
                if tp_size > 1:
                    self._connect_tp()
                    assert cfg.vocab % tp_size == 0
                    self.lm_rows = cfg.vocab // tp_size
                    self.lm_row0 = tp_rank * self.lm_rows
                self.plan = ctx.decode_plan(
                    [dict(qkv=self.wqkv[l].handle, o=self.wo[l].handle, gate_up=self.wgu[l].handle,
                          down=self.wdown[l].handle, gamma_attn=self.gamma.data_ptr(),
                          gamma_mlp=self.gamma.data_ptr(), kcache=self.kcache[l].data_ptr(),
                          vcache=self.vcache[l].data_ptr(),
                          kscale=self.kscale[l].data_ptr() if kv_int8 else None,
                          vscale=self.vscale[l].data_ptr() if kv_int8 else None) for l in range(self.n_layers)],
                    cfg.hidden, self.mlp_l, self.nq_l, self.nkv_l, cfg.head_dim, max_seq, cfg.eps, cfg.rope_theta,
                    tp=self.tp_comm, kv_int8=kv_int8, batch=batch, **(plan_options or {}))
            except YscvCudaError as e:
                if e.status != -3:  # anything but "unsupported shape" is a real failure
                    raise
            if tp_size > 1:
                import torch.distributed as dist
                ok = torch.tensor([1 if self.plan is not None else 0], device=self.dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.pg)
                if int(ok.item()) == 0 and self.plan is not None:
                    self.plan.free()
                    self.plan = None

    def _connect_tp(self):
        """Create this rank's exchange region, gather every rank's IPC handle, map the peers."""
        import numpy as np
        import torch.distributed as dist
        self.tp_comm = TpComm(self.ctx, self.tp_rank, self.tp_size, self.cfg.hidden)
        mine = torch.from_numpy(self.tp_comm.handle_bytes.copy()).to(self.dev)
        gathered = [torch.empty_like(mine) for _ in range(self.tp_size)]
        dist.all_gather(gathered, mine, group=self.pg)
        self.tp_comm.connect(np.stack([g.cpu().numpy() for g in gathered]))
        dist.barrier(group=self.pg)  # every region is mapped everywhere before anyone stores into one

    # ---- weights -------------------------------------------------------------------
    def _normal(self, tag: int, rows: int, cols: int) -> torch.Tensor:
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(self.seed * 1_000_003 + tag)
        return torch.randn(rows, cols, device=self.dev, generator=gen) * self.cfg.weight_std

    def _pack(self, w: torch.Tensor):
        n, k = w.shape
        g = self.cfg.group_size
        packed = torch.empty(n, k // 2, dtype=torch.uint8, device=self.dev)
        scales = torch.empty(n, k // g, dtype=torch.float32, device=self.dev)
        self.ctx.pack_int4_dev(w.data_ptr(), n, k, g, packed.data_ptr(), scales.data_ptr())
        return packed, scales

    def _linear(self, packed, scales) -> Int4Linear:
        packed, scales = packed.contiguous(), scales.contiguous()
        return Int4Linear(self.ctx, packed, scales, packed.shape[0], packed.shape[1] * 2, self.cfg.group_size)

    def _build_weights(self, keep_full: bool = False):
        c, r, G = self.cfg, self.tp_rank, self.tp_size
        d, H = c.head_dim, c.hidden
        self.embedding = self._normal(1, c.vocab, H)
        self.lm_head = self._normal(2, c.vocab, H)
        self.gamma = torch.ones(H, device=self.dev)
        self.wqkv, self.wo, self.wgu, self.wdown = [], [], [], []
        for l in range(self.n_layers):
            base = 100 * (l + 1)
            # fused rows: all q heads, then k heads, then v heads (each [heads*d, H])
            pq, sq = self._pack(self._normal(base + 1, c.n_q * d, H))
            pk, sk = self._pack(self._normal(base + 2, c.n_kv * d, H))
            pv, sv = self._pack(self._normal(base + 3, c.n_kv * d, H))
            po, so = self._pack(self._normal(base + 4, H, c.n_q * d))
            pg, sg = self._pack(self._normal(base + 5, c.mlp, H))
            pu, su = self._pack(self._normal(base + 6, c.mlp, H))
            pd, sd = self._pack(self._normal(base + 7, H, c.mlp))
            if self._keep_full:
                self.full[l] = dict(q=(pq, sq), k=(pk, sk), v=(pv, sv), o=(po, so), gate=(pg, sg), up=(pu, su),
                                    down=(pd, sd))
            # column-parallel: this rank's q heads, kv heads, gate and up rows; row-parallel: its
            # K slice of the output and down projections
            g = c.group_size
            parts = [sharding.shard_rows(pq, sq, r, G), sharding.shard_rows(pk, sk, r, G),
                     sharding.shard_rows(pv, sv, r, G)]
            self.wqkv.append(self._linear(torch.cat([p for p, _ in parts]), torch.cat([s for _, s in parts])))
            self.wo.append(self._linear(*sharding.shard_cols(po, so, g, r, G)))
            parts = [sharding.shard_rows(pg, sg, r, G), sharding.shard_rows(pu, su, r, G)]
            self.wgu.append(self._linear(torch.cat([p for p, _ in parts]), torch.cat([s for _, s in parts])))
            self.wdown.append(self._linear(*sharding.shard_cols(pd, sd, g, r, G)))

    _keep_full = False

    @classmethod
    def with_full_weights(cls, *args, **kw):
        """Same decoder, but the unsharded packed weights stay available in `.full`
        (the parity tests read them back to the host)."""
        class _Keep(cls):
            _keep_full = True
        return _Keep(*args, **kw)

    # ---- forward -------------------------------------------------------------------
    def _buf(self, name, *shape, dtype=torch.float32):
        key = (name, shape, dtype)
        if key not in self._bufs:
            self._bufs[key] = torch.empty(*shape, dtype=dtype, device=self.dev)
        return self._bufs[key]

    def _all_reduce(self, t: torch.Tensor):
        if self.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.pg)

    def forward(self, tokens: torch.Tensor, seq: int) -> torch.Tensor:
        """tokens: int32 [batch*seq] on the device (row b*seq + s). Runs the whole stack at
        positions *pos .. *pos+seq-1, leaves the greedy next token of every sequence in
        self.next_tokens, advances *pos by seq, and returns the logits [batch, vocab]."""
        c, ctx, B = self.cfg, self.ctx, self.batch
        H, d = c.hidden, c.head_dim
        rows = B * seq
        qkv_w = (self.nq_l + 2 * self.nkv_l) * d
        x = self._buf("x", rows, H)
        h = self._buf("h", rows, H)
        qkv = self._buf("qkv", rows, qkv_w)
        attn = self._buf("attn", rows, self.nq_l * d)
        o = self._buf("o", rows, H)
        gu = self._buf("gu", rows, 2 * self.mlp_l)
        act = self._buf("act", rows, self.mlp_l)
        down = self._buf("down", rows, H)
        # more than 16 rows take the tensor-core GEMM, whose bf16 activations the norm and SwiGLU kernels
        # can write themselves (one launch less in front of the QKV, gate/up and down projections)
        act16 = rows > 16 and not ctx.prefill_exact and H % 64 == 0 and self.mlp_l % 64 == 0
        if act16:
            h16 = self._buf("h16", rows, H, dtype=torch.bfloat16)
            a16 = self._buf("a16", rows, self.mlp_l, dtype=torch.bfloat16)
        fused = self.plan is not None and seq == 1
        if fused:
            # the whole step in one launch: layers, final norm, LM head, greedy token, position
            logits = self._buf("logits", B, c.vocab)
            if tokens.data_ptr() != self.next_tokens.data_ptr():
                self.next_tokens.copy_(tokens)
            # (tensor parallel: this rank's rows of the LM head; `logits` then holds only those)
            self.plan.step_token_shard_dev(self.embedding.data_ptr(), c.vocab, self.next_tokens.data_ptr(),
                                           self.pos.data_ptr(), self.gamma.data_ptr(),
                                           self.lm_head.data_ptr() + self.lm_row0 * H * 4, self.lm_row0, self.lm_rows,
                                           x.data_ptr(), logits.data_ptr())
            return logits
        ctx.embedding_dev(self.embedding.data_ptr(), c.vocab, H, tokens.data_ptr(), rows, x.data_ptr())
        delta = 0
        for l in range(self.n_layers):
            if act16:
                ctx.add_rms_norm_act_dev(x.data_ptr(), delta, self.gamma.data_ptr(), c.eps, rows, H, x.data_ptr(), h16.data_ptr())
                ctx.int4_matmul_act_dev(self.wqkv[l].handle, h16.data_ptr(), qkv.data_ptr(), rows)
            else:
                ctx.add_rms_norm_dev(x.data_ptr(), delta, self.gamma.data_ptr(), c.eps, rows, H, x.data_ptr(), h.data_ptr())
                ctx.int4_matmul_dev(self.wqkv[l].handle, h.data_ptr(), qkv.data_ptr(), rows)
            if self.kv_int8:
                ctx.rope_kv_append_i8_dev(qkv.data_ptr(), B, seq, self.nq_l, self.nkv_l, d, c.rope_theta,
                                          self.pos.data_ptr(), self.kcache[l].data_ptr(), self.kscale[l].data_ptr(),
                                          self.vcache[l].data_ptr(), self.vscale[l].data_ptr(), self.max_seq)
                ctx.gqa_attention_i8_dev(qkv.data_ptr(), qkv_w, B, seq, self.nq_l, self.nkv_l, d,
                                         self.kcache[l].data_ptr(), self.kscale[l].data_ptr(),
                                         self.vcache[l].data_ptr(), self.vscale[l].data_ptr(), self.max_seq,
                                         self.pos.data_ptr(), True, attn.data_ptr())
            else:
                ctx.rope_kv_append_dev(qkv.data_ptr(), B, seq, self.nq_l, self.nkv_l, d, c.rope_theta, self.pos.data_ptr(),
                                       self.kcache[l].data_ptr(), self.vcache[l].data_ptr(), self.max_seq)
                ctx.gqa_attention_dev(qkv.data_ptr(), qkv_w, B, seq, self.nq_l, self.nkv_l, d, self.kcache[l].data_ptr(),
                                      self.vcache[l].data_ptr(), self.max_seq, self.pos.data_ptr(), True, attn.data_ptr())
            ctx.int4_matmul_dev(self.wo[l].handle, attn.data_ptr(), o.data_ptr(), rows)
            self._all_reduce(o)
            if act16:
                ctx.add_rms_norm_act_dev(x.data_ptr(), o.data_ptr(), self.gamma.data_ptr(), c.eps, rows, H, x.data_ptr(), h16.data_ptr())
                ctx.int4_matmul_act_dev(self.wgu[l].handle, h16.data_ptr(), gu.data_ptr(), rows)
                ctx.swiglu_act_dev(gu.data_ptr(), rows, self.mlp_l, a16.data_ptr())
                ctx.int4_matmul_act_dev(self.wdown[l].handle, a16.data_ptr(), down.data_ptr(), rows)
            else:
                ctx.add_rms_norm_dev(x.data_ptr(), o.data_ptr(), self.gamma.data_ptr(), c.eps, rows, H, x.data_ptr(), h.data_ptr())
                ctx.int4_matmul_dev(self.wgu[l].handle, h.data_ptr(), gu.data_ptr(), rows)
                ctx.swiglu_dev(gu.data_ptr(), rows, self.mlp_l, act.data_ptr())
                ctx.int4_matmul_dev(self.wdown[l].handle, act.data_ptr(), down.data_ptr(), rows)
            self._all_reduce(down)
            delta = down.data_ptr()
        ctx.add_rms_norm_dev(x.data_ptr(), delta, self.gamma.data_ptr(), c.eps, rows, H, x.data_ptr(), h.data_ptr())
        last = h if seq == 1 else h.view(B, seq, H)[:, seq - 1, :].contiguous()
        logits = self._buf("logits", B, c.vocab)
        ctx.f32_matmul_dev(self.lm_head.data_ptr(), last.data_ptr(), B, c.vocab, H, logits.data_ptr())
        ctx.argmax_last_dev(logits.data_ptr(), B, c.vocab, self.next_tokens.data_ptr())
        ctx.advance_pos_dev(self.pos.data_ptr(), seq)
        return logits

    def close(self):
        """Drop the captured graph and every device buffer. With tensor parallelism call this
        before the process group is destroyed: a graph that holds NCCL nodes must go first."""
        self.stream.synchronize()
        self.graph = None
        if self.plan is not None:
            self.plan.free()
            self.plan = None
        if self.tp_comm is not None:
            # no rank may unmap a region a peer's kernel could still be storing into
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.pg)
            self.tp_comm.close()
            self.tp_comm = None
        self._bufs.clear()
        self.kcache, self.vcache = [], []
        self.wqkv, self.wo, self.wgu, self.wdown = [], [], [], []
        torch.cuda.synchronize()

    # ---- the llm-bench loop: prefill, then greedy decode with the KV cache -------------
    def reset(self):
        with torch.cuda.stream(self.stream):
            self.pos.zero_()

    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """prompt: int32 [batch, prompt_len] on the device."""
        with torch.cuda.stream(self.stream):
            return self.forward(prompt.reshape(-1).contiguous(), prompt.shape[1])

    def capture_decode_step(self):
        """Record one decode step (reads self.next_tokens, writes it back) as a CUDA graph."""
        with torch.cuda.stream(self.stream):
            saved = self.pos.clone(), self.next_tokens.clone()
            self.forward(self.next_tokens, 1)  # warm-up: sizes every buffer outside the capture
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream, capture_error_mode="thread_local"):
                self.forward(self.next_tokens, 1)
            self.pos.copy_(saved[0])
            self.next_tokens.copy_(saved[1])
        self.stream.synchronize()
        self.graph = g

    def decode(self, steps: int, use_graph: bool = True) -> torch.Tensor:
        """`steps` single-token passes after a prefill, each fed the previous pass's greedy
        token (the first one is fed the token the prefill chose). Returns the tokens the
        passes produced, int32 [steps, batch]. The work is enqueued on the decoder's stream:
        synchronise it before reading the result."""
        out = torch.empty(steps, self.batch, dtype=torch.int32, device=self.dev)
        with torch.cuda.stream(self.stream):
            for i in range(steps):
                if use_graph and self.graph is not None:
                    self.graph.replay()
                else:
                    self.forward(self.next_tokens, 1)
                out[i].copy_(self.next_tokens)
        return out
