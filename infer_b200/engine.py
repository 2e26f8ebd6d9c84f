"""The paged KV path driven the way the reference engine drives it, with synthetic weights.

The reference's loop is ``LLMEngine.step``: ``Scheduler.schedule`` picks a prefill batch or a
decode batch, ``ModelRunner.run`` builds the step metadata and runs the model (decode through
CUDA graphs captured per batch-size bucket over zero-filled static buffers), and
``Scheduler.postprocess`` appends the sampled tokens and frees finished requests
(infer/engine/llm_engine.py:37-82, infer/engine/scheduler.py:22-70,
infer/engine/model_runner.py:128-198).  Model weights are not available where this package
is built, so the model here is ONE attention layer with random weights: embedding, fused qkv
projection, per-head q/k RMSNorm, rotary embedding, the paged attention of this package,
output projection, logits, greedy sampling.  The projections and the norm/rotation run in
PyTorch (they are outside the path this package replaces); the KV append and the attention
run through ``infer_b200.attention.Attention``, i.e. through the sm_100a kernels.

``Scheduler`` follows the reference's policy, including preemption
(infer/engine/scheduler.py:44-61: when a running request cannot grow, the most recently
admitted one gives its pages back and returns to the front of the waiting queue).

One deliberate difference from the reference's capture scheme: the reference zero-fills its
static buffers before every replay, so the padding rows of a bucket carry slot 0 and its store
kernel overwrites slot 0 of page 0 with the padding row's k/v.  Here the padding rows carry
slot -1, which the append kernels skip, and context length 0, which the attention kernels skip.
"""
from __future__ import annotations

from collections import deque

import torch

from . import metadata
from .attention import Attention
from .block_manager import BlockManager
from .context import get_context, reset_context, set_context
from .sequence import Sequence


class Scheduler:
    def __init__(self, num_blocks: int, block_size: int, max_num_seqs: int = 64, max_num_batched_tokens: int = 32768):
        self.max_num_seqs, self.max_num_batched_tokens = max_num_seqs, max_num_batched_tokens
        self.block_manager = BlockManager(num_blocks, block_size)
        self.waiting: deque = deque()
        self.running: deque = deque()
        self.preemptions = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    def schedule(self):
        """-> (sequences, is_prefill).  Waiting requests are admitted first (as many as fit);
        otherwise every running request takes one decode step, preempting from the back of the
        queue when the pool cannot give a growing request its next page."""
        batch, tokens = [], 0
        while self.waiting and len(batch) < self.max_num_seqs:
            seq = self.waiting[0]
            if tokens + len(seq) > self.max_num_batched_tokens or not self.block_manager.can_allocate(seq):
                break
            self.block_manager.allocate(seq)
            tokens += len(seq) - seq.num_cached_tokens
            self.waiting.popleft()
            self.running.append(seq)
            batch.append(seq)
        if batch:
            return batch, True
        while self.running and len(batch) < self.max_num_seqs:
            seq = self.running.popleft()
            admitted = True
            while not self.block_manager.can_append(seq):
                if self.running:
                    self.preempt(self.running.pop())
                else:
                    self.preempt(seq)
                    admitted = False
                    break
            if admitted:
                self.block_manager.may_append(seq)
                batch.append(seq)
        if not batch:
            raise RuntimeError("Scheduler: the page pool cannot hold a single request")
        self.running.extendleft(reversed(batch))
        return batch, False

    def preempt(self, seq: Sequence):
        self.block_manager.deallocate(seq)
        self.waiting.appendleft(seq)
        self.preemptions += 1

    def postprocess(self, seqs, token_ids):
        for seq, tok in zip(seqs, token_ids):
            seq.append_token(tok)
            if seq.num_completion_tokens >= seq.max_tokens:
                self.block_manager.deallocate(seq)
                self.running.remove(seq)


class AttentionLayerModel(torch.nn.Module):
    """Embedding -> qkv projection -> q/k RMSNorm -> rotary embedding -> paged attention -> output
    projection; ``compute_logits`` turns the hidden state into vocabulary scores.  Random bf16
    weights from a seeded generator."""

    def __init__(self, hidden: int, n_q_heads: int, n_kv_heads: int, vocab: int, max_position: int, device, seed: int = 0,
                 eps: float = 1e-6):
        super().__init__()
        d = 128
        gen = torch.Generator().manual_seed(seed)
        rnd = lambda *shape, s=1.0: (torch.randn(*shape, generator=gen) * s).bfloat16().to(device)
        self.hidden, self.n_q_heads, self.n_kv_heads, self.eps = hidden, n_q_heads, n_kv_heads, eps
        self.embed = rnd(vocab, hidden)
        self.w_qkv = rnd(hidden, (n_q_heads + 2 * n_kv_heads) * d, s=hidden ** -0.5)
        self.w_o = rnd(n_q_heads * d, hidden, s=(n_q_heads * d) ** -0.5)
        self.w_head = rnd(hidden, vocab, s=hidden ** -0.5)
        self.q_norm_w = (1 + 0.1 * torch.randn(d, generator=gen)).bfloat16().to(device)
        self.k_norm_w = (1 + 0.1 * torch.randn(d, generator=gen)).bfloat16().to(device)
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
        ang = torch.arange(max_position).float()[:, None] * inv_freq[None]
        self.cos, self.sin = ang.cos().bfloat16().to(device), ang.sin().bfloat16().to(device)
        self.attn = Attention(n_q_heads, d, d ** -0.5, n_kv_heads)
        self.tap = None            # when a dict: receives the tensors handed to / returned by the attention path

    def _norm_rope(self, x, weight, positions):
        dt = x.dtype
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        x = xf.to(dt) * weight
        cos, sin = self.cos[positions][:, None, :], self.sin[positions][:, None, :]
        x1, x2 = x.chunk(2, dim=-1)
        return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)

    def forward(self, input_ids, positions):
        d, hq, hkv = 128, self.n_q_heads, self.n_kv_heads
        x = self.embed[input_ids]
        qkv = x @ self.w_qkv
        q = self._norm_rope(qkv[:, :hq * d].reshape(-1, hq, d), self.q_norm_w, positions)
        k = self._norm_rope(qkv[:, hq * d:(hq + hkv) * d].reshape(-1, hkv, d), self.k_norm_w, positions)
        v = qkv[:, (hq + hkv) * d:].reshape(-1, hkv, d).contiguous()
        o = self.attn(q, k, v)
        if self.tap is not None:
            self.tap.update(q=q, k=k, v=v, o=o)
        return x + o @ self.w_o

    def compute_logits(self, hidden):
        return hidden @ self.w_head


class LayerRunner:
    """The reference's ``ModelRunner`` for the one-layer model: page pools, step metadata, eager
    prefill, decode through per-bucket CUDA graphs over static buffers."""

    def __init__(self, model: AttentionLayerModel, num_blocks: int, block_size: int, max_num_seqs: int, max_model_len: int,
                 device, enforce_eager: bool = False, device_metadata: bool = False):
        """``device_metadata``: keep the decode step's metadata on the GPU (``metadata.DecodeState``): while the
        batch keeps its composition a step costs one small kernel (lengths + 1, slots and positions from the block
        tables already on the device) and the upload of newly allocated page ids, instead of the reference's
        per-step rebuild and upload (infer/engine/model_runner.py:110-126); the graphs read the state's tensors."""
        self.model, self.block_size, self.device, self.enforce_eager = model, block_size, torch.device(device), enforce_eager
        self.max_num_seqs, self.max_pages = max_num_seqs, -(-max_model_len // block_size)
        self.state = None
        if device_metadata and not enforce_eager:
            self.state = metadata.DecodeState(min(max_num_seqs, 512), self.max_pages, block_size, self.device)
            self._state_ids, self._state_lens = None, None
        # one zero-filled tensor [2, num_blocks, block_size, Hkv, 128]; the layer gets its two halves
        self.kv_cache = torch.zeros(2, num_blocks, block_size, model.n_kv_heads, 128, dtype=torch.bfloat16, device=device)
        model.attn.k_cache, model.attn.v_cache = self.kv_cache[0], self.kv_cache[1]
        self.graphs, self.graph_taps, self.graph_bs = {}, {}, []
        self.last_tap, self.last_bucket = None, None
        if not enforce_eager:
            self.capture_cudagraph()

    @torch.inference_mode()
    def capture_cudagraph(self):
        max_bs = min(self.max_num_seqs, 512)
        dev = self.device
        self.vars = dict(
            input_ids=torch.zeros(max_bs, dtype=torch.int64, device=dev),
            positions=torch.zeros(max_bs, dtype=torch.int64, device=dev),
            slot_mapping=torch.full((max_bs,), -1, dtype=torch.int32, device=dev),
            context_lens=torch.zeros(max_bs, dtype=torch.int32, device=dev),
            block_tables=torch.zeros(max_bs, self.max_pages, dtype=torch.int32, device=dev),
            outputs=torch.zeros(max_bs, self.model.hidden, dtype=torch.bfloat16, device=dev))
        v = self.vars
        if self.state is not None:                 # the graphs read the device-resident state directly
            v.update(positions=self.state.positions, slot_mapping=self.state.slot_mapping,
                     context_lens=self.state.context_lens, block_tables=self.state.block_tables)
        self.graph_bs = [b for b in [1, 2, 4, 8] if b <= max_bs] + list(range(16, max_bs + 1, 16))
        pool = None
        for bs in reversed(self.graph_bs):
            graph = torch.cuda.CUDAGraph()
            set_context(False, slot_mapping=v["slot_mapping"][:bs], context_lens=v["context_lens"][:bs],
                        block_tables=v["block_tables"][:bs])
            self.model.tap = None
            v["outputs"][:bs] = self.model(v["input_ids"][:bs], v["positions"][:bs])          # warm-up: sizes every scratch buffer
            self.model.tap = tap = {}
            with torch.cuda.graph(graph, pool):
                v["outputs"][:bs] = self.model(v["input_ids"][:bs], v["positions"][:bs])
            self.model.tap = None
            pool = pool or graph.pool()
            self.graphs[bs], self.graph_taps[bs] = graph, tap                                  # the tapped tensors stay alive with the graph
            torch.cuda.synchronize()
            reset_context()

    @torch.inference_mode()
    def run_model(self, input_ids, positions, is_prefill: bool):
        n = input_ids.numel()
        if is_prefill or self.enforce_eager or n > 512:
            self.model.tap = tap = {}
            hidden = self.model(input_ids, positions)
            self.model.tap = None
            self.last_tap, self.last_bucket = tap, None
            return self.model.compute_logits(hidden)
        ctx = get_context()
        bs = next(b for b in self.graph_bs if b >= n)
        v = self.vars
        if self.state is not None:                 # metadata already in place (run() advanced the state)
            v["input_ids"][:n] = input_ids
            self.graphs[bs].replay()
            self.last_tap, self.last_bucket = self.graph_taps[bs], bs
            return self.model.compute_logits(v["outputs"][:n])
        for name, t in v.items():
            if name == "slot_mapping":
                t.fill_(-1)
            elif name != "outputs":
                t.zero_()
        v["input_ids"][:n] = input_ids
        v["positions"][:n] = positions
        v["slot_mapping"][:n] = ctx.slot_mapping
        v["context_lens"][:n] = ctx.context_lens
        v["block_tables"][:n, :ctx.block_tables.size(1)] = ctx.block_tables
        self.graphs[bs].replay()
        self.last_tap, self.last_bucket = self.graph_taps[bs], bs
        return self.model.compute_logits(v["outputs"][:n])

    def run(self, seqs, is_prefill: bool):
        """-> sampled token ids (greedy).  Prefill always publishes block tables: the keys are read from
        the pools, also when no prefix is cached."""
        if is_prefill:
            input_ids, positions = metadata.prepare_prefill(seqs, self.block_size, self.device)
            ctx = get_context()
            if ctx.block_tables is None:
                ctx.block_tables = metadata.prepare_block_tables(seqs, self.device)
        elif self.state is not None and len(seqs) <= 512:
            ids, lens = [s.seq_id for s in seqs], [len(s) for s in seqs]
            if ids == self._state_ids and lens == [n + 1 for n in self._state_lens]:
                self.state.publish_new_pages(seqs)
            else:                                  # new composition (a request finished, arrived or was preempted)
                self.state.load(seqs, pending=1)
            self.state.advance()                   # also publishes the Context
            self._state_ids, self._state_lens = ids, lens
            n = len(seqs)
            ctx = get_context()
            ctx.slot_mapping, ctx.context_lens = self.state.slot_mapping[:n], self.state.context_lens[:n]
            ctx.block_tables = self.state.block_tables[:n]
            input_ids = torch.tensor([s.last_token for s in seqs], dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            positions = self.state.positions[:n]
        else:
            input_ids, positions = metadata.prepare_decode(seqs, self.block_size, self.device)
        logits = self.run_model(input_ids, positions, is_prefill)
        if is_prefill:
            last = get_context().cu_seqlens_q[1:].long() - 1
            logits = logits[last]
        tokens = logits.float().argmax(dim=-1).tolist()
        return tokens


class Engine:
    """``LLMEngine.step`` for the one-layer model: schedule, run, postprocess."""

    def __init__(self, runner: LayerRunner, scheduler: Scheduler):
        self.runner, self.scheduler = runner, scheduler
        self.steps = 0

    def add_request(self, token_ids, max_tokens: int) -> Sequence:
        seq = Sequence(token_ids, max_tokens=max_tokens)
        self.scheduler.add(seq)
        return seq

    def step(self):
        """-> (sequences of the step, is_prefill, sampled tokens); the step's Context is left in place
        for the caller to inspect and must be cleared with ``reset_context()``."""
        seqs, is_prefill = self.scheduler.schedule()
        tokens = self.runner.run(seqs, is_prefill)
        self.scheduler.postprocess(seqs, tokens)
        self.steps += 1
        return seqs, is_prefill, tokens
