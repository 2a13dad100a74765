"""The part of the model runner that hosts the tensor-parallel layer path.

It covers what nanovllm/engine/model_runner.py does around the model on each
rank: runtime set-up between device selection and model construction (:26-31),
KV-cache allocation and binding (:103-121), batch -> tensors for prefill and
decode (:123-188), CUDA-graph capture and replay for decode (:195-212,
:222-257) and teardown order (:50-59).  The scheduler, block manager,
tokenizer and the shared-memory RPC between ranks stay outside: callers hand
in token lists and block tables (every rank must be given the same batch).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..layers.sampler import Sampler
from ..models.qwen3 import Qwen3ForCausalLM
from ..runtime import get_runtime, init_runtime, shutdown_runtime
from ..utils.context import reset_context, set_context

FUSED_SAMPLER_MAX_ROWS = 256  # b2_lm_head_sample takes one token tile of the feature-lane layout


@dataclass
class ModelConfig:
    """The fields of a HF Qwen3 config the model reads (nanovllm/models/qwen3.py:127-143,167-171,199-203)."""
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    num_hidden_layers: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    rope_scaling: dict | None = None


QWEN3_0_6B = dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                  num_hidden_layers=28, vocab_size=151936, tie_word_embeddings=True)
QWEN3_8B = dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                num_hidden_layers=36, vocab_size=151936, tie_word_embeddings=False)
QWEN3_32B = dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600,
                 num_hidden_layers=64, vocab_size=151936, tie_word_embeddings=False)


@dataclass
class Seq:
    """Minimal per-request state: the token ids so far, the KV blocks they
    occupy and how many leading tokens are already in the cache."""
    token_ids: list[int]
    block_table: list[int] = field(default_factory=list)
    num_cached_tokens: int = 0

    def __len__(self):
        return len(self.token_ids)


def random_init_(model: torch.nn.Module, seed: int, tp_rank: int) -> None:
    """Seeded N(0, 0.02) weights generated on the device (norm weights stay 1).
    Each rank draws its own shard: enough for throughput runs, where only the
    shapes matter; parity tests load shards of one full model instead."""
    g = torch.Generator(device="cuda").manual_seed(seed * 1000 + tp_rank)
    for name, p in model.named_parameters():
        if "norm" in name:
            p.data.fill_(1.0)
        else:
            p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0, 0.02, generator=g))


class ModelRunner:

    def __init__(self, config: ModelConfig, *, max_num_seqs: int = 512, max_model_len: int = 4096, max_num_batched_tokens: int = 16384,
                 kvcache_block_size: int = 256, num_kvcache_blocks: int | None = None, gpu_memory_utilization: float = 0.9,
                 enforce_eager: bool = False, oneshot_tokens: int = 1024, timeout_ms: int = 5000, seed: int = 0,
                 full_weights: dict | None = None, fused_sampler: bool | None = None, sample_seed: int = 0):
        assert dist.is_initialized(), "create the process group first (world size 1 included), as the reference does"
        self.config = config
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.block_size = kvcache_block_size
        self.max_num_seqs, self.max_model_len, self.max_num_batched_tokens = max_num_seqs, max_model_len, max_num_batched_tokens
        self.enforce_eager = enforce_eager
        # LM head and sampler in one pass (no [B, vocab] logits, no gather): the default at every world size
        if fused_sampler is None:
            fused_sampler = True
        self.fused_sampler = fused_sampler
        self.sample_seed = sample_seed
        self.device = torch.device("cuda", torch.cuda.current_device())
        # symmetric buffers exist before the layers are built, so graph capture sees fixed addresses
        self.runtime = init_runtime(max_tokens=max_num_batched_tokens, hidden=config.hidden_size, oneshot_tokens=oneshot_tokens,
                                    vocab=config.vocab_size, max_seqs=max_num_seqs, timeout_ms=timeout_ms)
        prev_dtype = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        torch.set_default_device(self.device)
        try:
            self.model = Qwen3ForCausalLM(config)
            if full_weights is not None:
                self.model.load_full_weights(full_weights)
            else:
                random_init_(self.model, seed, self.rank)
            self.sampler = Sampler()
            self._allocate_kv_cache(num_kvcache_blocks, gpu_memory_utilization)
            self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
            if not enforce_eager:
                self._capture_graphs()
        finally:
            torch.set_default_device("cpu")
            torch.set_default_dtype(prev_dtype)

    # ---- teardown (reference :50-59) --------------------------------------
    def exit(self):
        self.graphs = {}
        self.graph_pool = None
        torch.cuda.synchronize()
        shutdown_runtime()

    # ---- KV cache (reference :103-121) -------------------------------------
    def _allocate_kv_cache(self, num_blocks: int | None, utilization: float):
        c = self.config
        self.num_kv_heads = c.num_key_value_heads // self.world
        block_bytes = 2 * c.num_hidden_layers * self.block_size * self.num_kv_heads * c.head_dim * 2
        if num_blocks is None:
            free, total = torch.cuda.mem_get_info()
            budget = int(total * utilization) - (total - free)
            # activations of the largest prefill step: a few [tokens, widest layer output] bf16 tensors
            widest = max(2 * c.intermediate_size // self.world, c.hidden_size, (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim // self.world)
            budget -= 6 * self.max_num_batched_tokens * widest * 2
            num_blocks = budget // block_bytes
        assert num_blocks > 0, "no memory left for the KV cache"
        self.num_kvcache_blocks = int(num_blocks)
        self.kv_cache = torch.zeros(2, c.num_hidden_layers, self.num_kvcache_blocks, self.block_size, self.num_kv_heads, c.head_dim,
                                    dtype=torch.bfloat16, device=self.device)
        for i, layer in enumerate(self.model.model.layers):
            layer.self_attn.attn.k_cache = self.kv_cache[0, i]
            layer.self_attn.attn.v_cache = self.kv_cache[1, i]

    # ---- batch -> tensors -----------------------------------------------------
    def _h2d(self, values, dtype):
        return torch.tensor(values, dtype=dtype, pin_memory=True).to(self.device, non_blocking=True)

    def _block_tables(self, seqs: list[Seq]):
        width = max(len(s.block_table) for s in seqs)
        return self._h2d([s.block_table + [-1] * (width - len(s.block_table)) for s in seqs], torch.int32)

    def prepare_prefill(self, seqs: list[Seq], num_new: list[int] | None = None):
        """Tokens [num_cached, num_cached + new) of each sequence are computed;
        their K/V go to the slots their block table assigns (reference :129-170)."""
        ids, pos, slots, cu_q, cu_k = [], [], [], [0], [0]
        max_q = max_k = 0
        bs = self.block_size
        for i, s in enumerate(seqs):
            start = s.num_cached_tokens
            end = len(s) if num_new is None else start + num_new[i]
            ids.extend(s.token_ids[start:end])
            pos.extend(range(start, end))
            cu_q.append(cu_q[-1] + end - start)
            cu_k.append(cu_k[-1] + end)
            max_q, max_k = max(max_q, end - start), max(max_k, end)
            if s.block_table:
                slots.extend(s.block_table[p // bs] * bs + p % bs for p in range(start, end))
        block_tables = self._block_tables(seqs) if cu_k[-1] > cu_q[-1] else None
        ids_t, pos_t = self._h2d(ids, torch.int64), self._h2d(pos, torch.int64)
        set_context(True, self._h2d(cu_q, torch.int32), self._h2d(cu_k, torch.int32), max_q, max_k,
                    self._h2d(slots, torch.int32) if slots else None, None, block_tables)
        return ids_t, pos_t

    def prepare_decode(self, seqs: list[Seq]):
        """One new token per sequence: the last one of its list (reference :172-188)."""
        bs = self.block_size
        ids = [s.token_ids[-1] for s in seqs]
        pos = [len(s) - 1 for s in seqs]
        slots = [s.block_table[(len(s) - 1) // bs] * bs + (len(s) - 1) % bs for s in seqs]
        lens = [len(s) for s in seqs]
        set_context(False, slot_mapping=self._h2d(slots, torch.int32), context_lens=self._h2d(lens, torch.int32),
                    block_tables=self._block_tables(seqs))
        return self._h2d(ids, torch.int64), self._h2d(pos, torch.int64)

    # ---- forward ---------------------------------------------------------------
    @torch.inference_mode()
    def run_model(self, input_ids: torch.Tensor, positions: torch.Tensor, is_prefill: bool):
        return self.model.compute_logits(self.run_hidden(input_ids, positions, is_prefill))

    def run_hidden(self, input_ids: torch.Tensor, positions: torch.Tensor, is_prefill: bool):
        """The model forward up to the final norm (eager for prefill, a graph replay for decode)."""
        from ..utils.context import get_context
        n = input_ids.size(0)
        if is_prefill or self.enforce_eager or n > self.graph_bs[-1]:
            return self.model(input_ids, positions)
        ctx = get_context()
        bs = next(b for b in self.graph_bs if b >= n)
        gv = self.graph_vars
        gv["input_ids"][:n] = input_ids
        gv["positions"][:n] = positions
        gv["slot_mapping"].fill_(-1)  # padded rows store nothing
        gv["slot_mapping"][:n] = ctx.slot_mapping
        gv["context_lens"].zero_()
        gv["context_lens"][:n] = ctx.context_lens
        gv["block_tables"][:n, :ctx.block_tables.size(1)] = ctx.block_tables
        self._bt_rows = {}  # the graph's table no longer matches what _decode_graph_step last staged
        self.graphs[bs].replay()
        return gv["outputs"][:n]

    def _decode_staging(self):
        """Pinned host mirrors of the graphs' input buffers, allocated once: a decode step fills them with
        numpy and issues one asynchronous copy per buffer straight into the graph's inputs (no per-step pinned
        allocations, no device-to-device staging copies)."""
        if getattr(self, "_stage", None) is None:
            gv = self.graph_vars
            self._stage = {k: torch.zeros(gv[k].shape, dtype=gv[k].dtype, pin_memory=True) for k in
                           ("input_ids", "positions", "slot_mapping", "context_lens", "block_tables")}
            self._stage_np = {k: v.numpy() for k, v in self._stage.items()}
            self._bt_rows = {}  # row of the staged block table -> the blocks last copied into the graph's table for it
        return self._stage, self._stage_np

    @torch.inference_mode()
    def _decode_graph_step(self, seqs: list[Seq]):
        """prepare_decode + the graph replay of run_model in one go, for batches a captured graph covers."""
        n = len(seqs)
        bs = next(b for b in self.graph_bs if b >= n)
        stage, np_ = self._decode_staging()
        blk = self.block_size
        lens = [len(s) for s in seqs]
        np_["input_ids"][:n] = [s.token_ids[-1] for s in seqs]
        np_["positions"][:n] = [l - 1 for l in lens]
        np_["context_lens"][:n] = lens
        np_["context_lens"][n:bs] = 0          # padded rows attend to nothing ...
        np_["slot_mapping"][:n] = [s.block_table[(l - 1) // blk] * blk + (l - 1) % blk for s, l in zip(seqs, lens)]
        np_["slot_mapping"][n:bs] = -1         # ... and store nothing
        # block tables change only when a sequence takes a new block (every 256 tokens) or the batch changes: rows are
        # rewritten, and the table copied, only then
        bt = np_["block_tables"]
        rows = self._bt_rows
        width, dirty = 0, False
        for i, s in enumerate(seqs):
            t = s.block_table
            width = max(width, len(t))
            key = tuple(t)
            if rows.get(i) != key:
                bt[i, :len(t)] = t
                rows[i] = key
                dirty = True
        gv = self.graph_vars
        for k in ("input_ids", "positions", "slot_mapping", "context_lens"):
            gv[k][:bs].copy_(stage[k][:bs], non_blocking=True)
        if dirty:
            gv["block_tables"][:n, :width].copy_(stage["block_tables"][:n, :width], non_blocking=True)
        self.graphs[bs].replay()
        set_context(False)  # the LM head only needs to know this is not a prefill step
        return gv["outputs"][:n]

    @torch.inference_mode()
    def step(self, seqs: list[Seq], is_prefill: bool, temperatures: list[float] | None = None, num_new: list[int] | None = None):
        """One forward pass + sampling on rank 0; the chosen token ids are
        returned on every rank.  temperatures=None means greedy (argmax)."""
        if not is_prefill and not self.enforce_eager and len(seqs) <= self.graph_bs[-1]:
            hidden = self._decode_graph_step(seqs)
        else:
            ids, pos = self.prepare_prefill(seqs, num_new) if is_prefill else self.prepare_decode(seqs)
            hidden = self.run_hidden(ids, pos, is_prefill)
        if getattr(self, "_picked", None) is None or self._picked.numel() < len(seqs):
            self._picked = torch.zeros(max(len(seqs), self.max_num_seqs), dtype=torch.int64, device=self.device)
        picked = self._picked[:len(seqs)]  # one buffer for every step: rank 0's sampler fills it, the broadcast hands it to the others
        if self.fused_sampler and len(seqs) <= FUSED_SAMPLER_MAX_ROWS:
            temps = None if temperatures is None else self._h2d(temperatures, torch.float32)
            self.model.sample_tokens(hidden, temps, self.sample_seed, out=picked)
        else:
            logits = self.model.compute_logits(hidden)
            if self.rank == 0:
                if temperatures is None:
                    picked = Sampler.greedy(logits)
                else:
                    picked = self.sampler(logits, self._h2d(temperatures, torch.float32))
        if self.world > 1:
            from .. import ops
            ops.broadcast_tokens(picked)  # rank 0's choice reaches every rank on the device
        tokens = picked.tolist()  # the step's synchronisation point
        reset_context()
        self.runtime.check_status()
        return tokens

    # ---- CUDA graphs (reference :222-257) -----------------------------------------
    @torch.inference_mode()
    def _capture_graphs(self):
        c = self.config
        max_bs = min(self.max_num_seqs, 512)
        max_blocks = (self.max_model_len + self.block_size - 1) // self.block_size
        dev = self.device
        gv = dict(
            input_ids=torch.zeros(max_bs, dtype=torch.int64, device=dev),
            positions=torch.zeros(max_bs, dtype=torch.int64, device=dev),
            slot_mapping=torch.full((max_bs,), -1, dtype=torch.int32, device=dev),
            context_lens=torch.zeros(max_bs, dtype=torch.int32, device=dev),
            block_tables=torch.zeros(max_bs, max_blocks, dtype=torch.int32, device=dev),
            outputs=torch.zeros(max_bs, c.hidden_size, dtype=torch.bfloat16, device=dev),
        )
        self.graph_bs = [b for b in (1, 2, 4, 8) if b <= max_bs] + list(range(16, max_bs + 1, 16))
        self.graph_pool = None
        for bs in reversed(self.graph_bs):
            graph = torch.cuda.CUDAGraph()
            set_context(False, slot_mapping=gv["slot_mapping"][:bs], context_lens=gv["context_lens"][:bs], block_tables=gv["block_tables"][:bs])
            gv["outputs"][:bs] = self.model(gv["input_ids"][:bs], gv["positions"][:bs])  # warm-up (also runs the collectives once)
            with torch.cuda.graph(graph, self.graph_pool):
                gv["outputs"][:bs] = self.model(gv["input_ids"][:bs], gv["positions"][:bs])
            if self.graph_pool is None:
                self.graph_pool = graph.pool()
            self.graphs[bs] = graph
            torch.cuda.synchronize()
            reset_context()
        self.graph_vars = gv


class ResidentDecoder:
    """Decode steps that never leave the device: one CUDA graph holds the model
    forward, the LM head with its gather, the greedy pick on rank 0, the token
    broadcast to the other ranks and the computation of the next step's inputs
    (what nanovllm/engine/model_runner.py:172-188 and :195-212 do with a host
    round trip every step).  `load(seqs)` puts a batch on the device;
    `replay()` advances every sequence by one token."""

    @torch.inference_mode()
    def __init__(self, runner: ModelRunner, batch: int):
        from .. import ops
        assert not runner.enforce_eager and batch in runner.graphs, "batch must be one of the captured decode batch sizes"
        self.r, self.bs, self.ops = runner, batch, ops
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=runner.device)
        gv = runner.graph_vars
        gv["slot_mapping"].fill_(-1)
        gv["context_lens"].zero_()
        before = ops._abi.launch_count()
        self._body()  # warm-up: also creates the logits view outside the capture
        self.kernels_per_step = ops._abi.launch_count() - before
        gv["slot_mapping"].fill_(-1)
        gv["context_lens"].zero_()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, runner.graph_pool):
            self._body()
        torch.cuda.synchronize()
        self.replays_left = 0  # nothing loaded yet

    @torch.inference_mode()
    def _body(self):
        r, bs, gv = self.r, self.bs, self.r.graph_vars
        set_context(False, slot_mapping=gv["slot_mapping"][:bs], context_lens=gv["context_lens"][:bs], block_tables=gv["block_tables"][:bs])
        hidden = r.model(gv["input_ids"][:bs], gv["positions"][:bs])
        if r.fused_sampler and bs <= FUSED_SAMPLER_MAX_ROWS:
            r.model.sample_tokens(hidden, None, r.sample_seed, out=self.tokens)  # greedy: rank 0 gets the picks
        else:
            logits = r.model.compute_logits(hidden)
            if r.rank == 0:
                self.ops.argmax(logits, self.tokens)
        if r.world > 1:
            self.ops.broadcast_tokens(self.tokens)
        self.ops.advance_decode(self.tokens, gv["input_ids"], gv["positions"], gv["context_lens"], gv["slot_mapping"],
                                gv["block_tables"][:bs], r.block_size, r.num_kvcache_blocks * r.block_size)
        reset_context()

    @torch.inference_mode()
    def load(self, seqs: list[Seq]) -> None:
        """The batch's state as prepare_decode would build it for the next step."""
        r, gv, n = self.r, self.r.graph_vars, len(seqs)
        assert n == self.bs
        bs = r.block_size
        width = max(len(s.block_table) for s in seqs)
        assert width <= gv["block_tables"].shape[1], "a block table is longer than max_model_len allows"
        assert all(len(s) <= len(s.block_table) * bs for s in seqs), "a sequence is longer than its block table"
        gv["input_ids"][:n] = r._h2d([s.token_ids[-1] for s in seqs], torch.int64)
        gv["positions"][:n] = r._h2d([len(s) - 1 for s in seqs], torch.int64)
        gv["context_lens"][:n] = r._h2d([len(s) for s in seqs], torch.int32)
        gv["slot_mapping"][:n] = r._h2d([s.block_table[(len(s) - 1) // bs] * bs + (len(s) - 1) % bs for s in seqs], torch.int32)
        r._bt_rows = {}  # the graph's table is rewritten here: _decode_graph_step must stage its rows again
        gv["block_tables"][:n].fill_(-1)  # columns past a sequence's own blocks: no room (the advance kernel freezes such a row)
        gv["block_tables"][:n, :width] = r._h2d([s.block_table + [-1] * (width - len(s.block_table)) for s in seqs], torch.int32)
        # replays until the first sequence has filled its last block: each replay stores the K/V of one more position
        self.replays_left = min(len(s.block_table) * bs - len(s) for s in seqs) + 1

    def replay(self) -> None:
        if self.replays_left <= 0:
            raise RuntimeError("ResidentDecoder.replay: a sequence has filled the blocks it was loaded with; load() a batch with more blocks")
        self.replays_left -= 1
        self.graph.replay()


def sequential_block_tables(lengths: list[int], block_size: int, first_block: int = 0, permutation: list[int] | None = None) -> list[list[int]]:
    """Block tables for sequences of the given (maximum) lengths, taking blocks
    in order from `first_block`, or from `permutation` (a shuffled free list)."""
    tables, nxt = [], first_block
    for n in lengths:
        need = (n + block_size - 1) // block_size
        ids = list(range(nxt, nxt + need))
        if permutation is not None:
            ids = [permutation[i] for i in ids]
        tables.append(ids)
        nxt += need
    return tables
