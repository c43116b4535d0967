"""Single-rank model runner of the engine shell (reference: core/model_runner.py:32-555).

What it keeps of the reference: prefill batches packed by a token budget (core/scheduler.py:65-108),
per-sequence retain budgets and PHI (utils/arguments.py:81-121), the global `Context` set before each
forward (:185-207,437-442), scoring + store on a side stream joined before decoding (:322-323),
page reclaim after a compressed prefill (:288-291), decode as CUDA-graph replays per padded batch
size with padding rows mapped to the reserved slot (:469-545), Gumbel-max sampling.

What it leaves out (control plane, out of scope): tokenizer / chat templates, HF weight loading,
multi-process tensor parallelism (`tensor_parallel_size` must be 1), preemption.
"""
from __future__ import annotations

import os
from collections import deque
from typing import List, Optional, Sequence as Seq, Tuple

import torch

from compactor_vllm.api_types import BatchCompressionParams, CompressionMethod
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.config.engine_config import LLMConfig
from compactor_vllm.core.memory_manager import KVCacheManager
from compactor_vllm.layers.sampler import Sampler
from compactor_vllm.models import MODEL_REGISTRY, registry_key
from compactor_vllm.utils import arguments as A
from compactor_vllm.utils.context import CompressionContext, reset_context, set_context
from compactor_vllm.utils.sequence import Sequence, SequenceStatus


def _pad_batch(n: int) -> int:
    """Captured batch sizes: powers of two (core/model_runner.py:99-107)."""
    b = 1
    while b < n:
        b *= 2
    return b


def _check_shape_envelope(hf, config: LLMConfig) -> None:
    """Fail at construction, with the reason, for geometries the sm_100a kernels do not serve (the per-call
    answer would be CVLLM_E_UNSUPPORTED in the middle of the first prefill)."""
    head_dim = getattr(hf, "head_dim", None) or hf.hidden_size // hf.num_attention_heads
    group = hf.num_attention_heads // hf.num_key_value_heads
    problems = []
    if head_dim != 128:
        problems.append(f"head_dim {head_dim} (only 128)")
    if group > 8:
        problems.append(f"GQA group {group} (decode serves <= 8)")
    if hf.num_key_value_heads > 16:
        problems.append(f"{hf.num_key_value_heads} KV heads per rank (selection serves <= 16)")
    if config.kvcache_page_size % 128 != 0:
        problems.append(f"kvcache_page_size {config.kvcache_page_size} (prefill needs a multiple of 128)")
    if config.leverage_sketch_size != 48:
        problems.append(f"leverage_sketch_size {config.leverage_sketch_size} (only 48)")
    if problems:
        raise ValueError("model / config outside the kernels' shape envelope: " + "; ".join(problems))


class KVCacheExhausted(RuntimeError):
    """The paged cache cannot hold the tokens a decode wave may still produce."""


class ModelRunner:
    def __init__(self, config: LLMConfig, *, num_pages: Optional[int] = None, seed: int = 0,
                 device_allocator: bool = True, max_batched_tokens: Optional[int] = None):
        assert config.tensor_parallel_size == 1, "the engine shell is single-rank (tensor parallelism: layers/linear.py)"
        assert torch.cuda.is_available(), "no CPU fallback"
        self.config = config
        hf = config.hf_config
        kind = registry_key(hf)
        self.mixed_steps = bool(getattr(MODEL_REGISTRY[kind], "mixed_steps", False))
        if not self.mixed_steps:
            _check_shape_envelope(hf, config)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.dtype = hf.torch_dtype if isinstance(hf.torch_dtype, torch.dtype) else torch.bfloat16
        if self.dtype not in ((torch.bfloat16, torch.float32) if self.mixed_steps else (torch.bfloat16, torch.float16)):
            raise ValueError(f"{kind} models do not run in {self.dtype}")
        if self.dtype == torch.float32:   # true 32-bit products: no reduced-precision matrix mode
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        prev = torch.get_default_dtype()
        torch.set_default_dtype(self.dtype)  # parameters are born in the model dtype on the GPU
        try:
            with torch.device(self.device):
                model = MODEL_REGISTRY[kind](hf)
        finally:
            torch.set_default_dtype(prev)
        weights = os.path.join(config.path, "model.safetensors") if config.path else None
        if weights and os.path.isfile(weights) and hasattr(model, "load_weights"):
            from compactor_vllm.utils.safetensors_io import load_safetensors

            model.load_weights(load_safetensors(weights))
        else:
            model.init_synthetic_weights(seed)
        self.model = model.to(self.device).eval()
        self.num_kv_heads = hf.num_key_value_heads
        self.head_dim = getattr(hf, "head_dim", None) or hf.hidden_size // hf.num_attention_heads
        self.kv = KVCacheManager(self.device.index, config)
        self.kv.head_dim = self.head_dim
        self.kv.model_dtype = self.dtype
        self.kv.init_cache(self.model, num_pages=num_pages, device_allocator=device_allocator)
        self.store_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.PHI = (None if self.mixed_steps
                    else A.make_phi(self.head_dim, config.leverage_sketch_size, self.dtype, self.device))
        self.sampler = Sampler()
        self.max_batched_tokens = int(max_batched_tokens or config.max_model_len)
        self.eos = config.eos
        self._graphs: dict = {}
        self._step_graphs: dict = {}
        self._room: dict = {}          # seq_id -> tokens the pages granted so far can hold (mixed-step models)
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "graph_replays": 0, "bytes_reclaimed": 0, "steps": 0}

    # ------------------------------------------------------------------ prefill
    def _prefill_batches(self, seqs: List[Sequence]) -> List[List[Sequence]]:
        batches, cur, tokens = [], [], 0
        for s in seqs:
            n = s.num_prompt_tokens
            assert 0 < n <= self.config.max_model_len, "prompt longer than max_model_len"
            if cur and (tokens + n > self.max_batched_tokens or len(cur) >= self.config.max_num_seqs):
                batches.append(cur)
                cur, tokens = [], 0
            cur.append(s)
            tokens += n
        if cur:
            batches.append(cur)
        return batches

    @torch.no_grad()
    def run_prefill(self, seqs: List[Sequence], params: BatchCompressionParams) -> torch.Tensor:
        dev = self.device
        lens = [s.num_prompt_tokens for s in seqs]
        ok, batch_mapping = self.kv.allocate_sequences([s.seq_id for s in seqs], lens)
        assert ok, "KV cache exhausted (no preemption in the engine shell)"
        ids = torch.tensor([t for s in seqs for t in s.prompt_token_ids], dtype=torch.int64, device=dev)
        positions = torch.cat([torch.arange(n, device=dev) for n in lens])
        cu = torch.zeros(len(seqs) + 1, dtype=torch.int32, device=dev)
        cu[1:] = torch.tensor(lens, dtype=torch.int32, device=dev).cumsum(0)
        ratios = [s.compression_params.compression_ratio for s in seqs]
        do_compression = (params.compression_method is not CompressionMethod.NONE
                          and any(r < 1.0 for r in ratios))
        cc = None
        if do_compression:
            first = [s.compression_params.protected_first_tokens for s in seqs]
            last = [s.compression_params.protected_last_tokens for s in seqs]
            retain = A.tokens_to_retain(lens, ratios, first, last, self.num_kv_heads)
            cc = CompressionContext(
                compression_method=params.compression_method,
                compression_chunk_size=params.chunk_size if params.do_chunked_compression else -1,
                batch_tokens_to_retain=torch.tensor(retain, dtype=torch.int32, device=dev),
                max_tokens_to_retain=A.max_tokens_to_retain(lens, self.num_kv_heads),
                context_lens=lens, PHI=self.PHI, protected_first_tokens=first, protected_last_tokens=last)
        set_context(is_prefill=True, do_compression=do_compression, cu_seqlens_q=cu, cu_seqlens_k=cu,
                    max_seqlen_q=max(lens), max_seqlen_k=max(lens), batch_mapping=batch_mapping,
                    max_bh_len=0, compression_context=cc, STORE_STREAM=self.store_stream)
        hidden = self.model(ids, positions)
        logits = self.model.compute_logits(hidden)
        reset_context()
        # scoring / selection / compaction ran beside attention; join before anything reads the cache
        torch.cuda.current_stream().wait_stream(self.store_stream)
        self.stats["prefill_tokens"] += sum(lens)
        if do_compression:  # give back the pages the evicted pairs no longer need (:288-291)
            self.stats["bytes_reclaimed"] += self.kv.reclaim_pages(
                [s.seq_id for s in seqs], [0] * len(seqs))
        return logits

    # ------------------------------------------------------------------- decode
    @torch.no_grad()
    def _decode_forward(self, ids, positions, batch_mapping, temps):
        set_context(is_prefill=False, batch_mapping=batch_mapping)
        hidden = self.model(ids, positions)
        logits = self.model.compute_logits(hidden)
        reset_context()
        return self.sampler(logits, temps)

    def _graph_for(self, bs: int):
        g = self._graphs.get(bs)
        if g is not None:
            return g
        dev = self.device
        st = {"ids": torch.zeros(bs, dtype=torch.int64, device=dev),
              "pos": torch.zeros(bs, dtype=torch.int64, device=dev),
              "bm": torch.full((bs,), RESERVED_BATCH, dtype=torch.int32, device=dev),
              "temps": torch.zeros(bs, dtype=torch.float32, device=dev)}
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            # warm-up on the capture stream with every row on the reserved slot: allocates the per-stream
            # workspaces and touches no sequence's cache
            self._decode_forward(st["ids"], st["pos"], st["bm"], st["temps"])
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                st["out"] = self._decode_forward(st["ids"], st["pos"], st["bm"], st["temps"])
        torch.cuda.current_stream().wait_stream(side)
        self._graphs[bs] = (graph, st)
        return self._graphs[bs]

    @torch.no_grad()
    def run_decode_loop(self, seqs: List[Sequence]) -> None:
        dev = self.device
        live = [s for s in seqs if s.status is SequenceStatus.RUNNING]
        if not live:
            return
        # capacity for every token this wave can still produce, reserved once (the reference reserves per
        # scheduler step on the host; `DevicePagedKVCache.reserve_tokens_device` is the in-graph alternative)
        for s in live:
            left = s.sampling_params.max_new_tokens - s.num_generated_tokens
            # never ask for more than the model length allows (generation stops there, see _accept): the tail
            # would be refused as "too long" although those tokens are never produced
            room = self.config.max_model_len - (s.num_prompt_tokens + s.num_generated_tokens)
            want = max(min(left, room), 0) + 1
            ok, _ = self.kv.allocate_sequences([s.seq_id], [want])
            if not ok:
                raise KVCacheExhausted(f"sequence {s.seq_id}: no room for {want} more tokens "
                                       f"({self.kv.num_free_pages} free pages; the engine shell has no preemption)")
        bs = _pad_batch(len(live))
        slots = [self.kv.seq_id_to_batch[s.seq_id] for s in live]
        bm = torch.full((bs,), RESERVED_BATCH, dtype=torch.int32, device=dev)
        bm[:len(live)] = torch.tensor(slots, dtype=torch.int32, device=dev)
        temps = torch.zeros(bs, dtype=torch.float32, device=dev)
        temps[:len(live)] = torch.tensor([s.sampling_params.temperature for s in live], device=dev)
        ids = torch.zeros(bs, dtype=torch.int64, device=dev)
        pos = torch.zeros(bs, dtype=torch.int64, device=dev)
        use_graph = not self.config.enforce_eager
        if use_graph:
            graph, st = self._graph_for(bs)
        while any(s.status is SequenceStatus.RUNNING for s in live):
            for i, s in enumerate(live):
                if s.status is SequenceStatus.RUNNING:
                    ids[i] = s.completion_token_ids[-1]
                    pos[i] = s.num_prompt_tokens + s.num_generated_tokens - 1
                else:
                    bm[i] = RESERVED_BATCH  # finished rows are skipped by the store and the attention
            if use_graph:
                st["ids"].copy_(ids); st["pos"].copy_(pos); st["bm"].copy_(bm); st["temps"].copy_(temps)
                graph.replay()
                out = st["out"]
                self.stats["graph_replays"] += 1
            else:
                out = self._decode_forward(ids, pos, bm, temps)
            self.stats["decode_steps"] += 1
            toks = out[:len(live)].tolist()
            for s, t in zip(live, toks):
                if s.status is SequenceStatus.RUNNING:
                    self._accept(s, t)

    def _accept(self, s: Sequence, token: int) -> None:
        s.add_new_token(token)
        full = s.num_prompt_tokens + s.num_generated_tokens >= self.config.max_model_len  # RoPE table / reservation
        if s.num_generated_tokens >= s.sampling_params.max_new_tokens or token == self.eos or full:
            s.status = SequenceStatus.FINISHED

    # -------------------------------------------------------------- mixed steps
    def _make_room(self, seq: Sequence, tokens: int) -> bool:
        """Cache room for `tokens` more tokens of a sequence (a slot at its first call).  What the pages already
        granted can hold is remembered on the host, so a step that stays inside it costs no allocator call and no
        device round trip - a decoding sequence asks once per page, or never when its whole length was reserved at
        admission."""
        need = seq.num_computed_tokens + tokens
        if need <= self._room.get(seq.seq_id, 0):
            return True
        ok, _ = self.kv.allocate_sequences([seq.seq_id], [tokens])
        if ok:
            ps = self.kv.page_size
            self._room[seq.seq_id] = max(self._room.get(seq.seq_id, 0), -(-need // ps) * ps)
        return ok

    @torch.no_grad()
    def run_step(self, entries: Seq[Tuple[Sequence, Seq[int]]], rows: Optional[Seq[int]] = None,
                 temperatures: Optional[Seq[float]] = None) -> torch.Tensor:
        """One forward pass over a mixed batch: every entry is (sequence, its next tokens) — a portion of a prompt
        or a single decoded token — continuing from what earlier steps left in the cache.  Returns the logits of
        `rows` (indices into the step's packed tokens; None = the last token of every entry), or — with
        `temperatures`, one per entry — the token sampled after every entry's last token.  Room for the new tokens
        is reserved here; a sequence gets its cache slot at its first entry.  Models with `mixed_steps`."""
        assert self.mixed_steps, "this model runs whole prompts and single tokens only"
        assert rows is None or temperatures is None
        dev = self.device
        lens = [len(t) for _, t in entries]
        assert lens and min(lens) > 0
        starts = [s.num_computed_tokens for s, _ in entries]
        for (s, _), n in zip(entries, lens):
            if not self._make_room(s, n):
                raise KVCacheExhausted(f"no room for {n} more tokens of sequence {s.seq_id} "
                                       f"({self.kv.num_free_tokens} tokens free)")
        T = sum(lens)
        if max(lens) == 1 and not self.config.enforce_eager:
            out = self._graph_decode_step(entries, starts, rows, temperatures)
            for s, _ in entries:
                s.num_computed_tokens += 1
            self.stats["steps"] += 1
            self.stats["graph_replays"] += 1
            return out
        # one host->device copy for all the step's index vectors
        pos = [p for st, n in zip(starts, lens) for p in range(st, st + n)]
        slot_of = [self.kv.seq_id_to_batch[s.seq_id] for s, _ in entries]
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        packed = torch.tensor([t for _, toks in entries for t in toks] + pos
                              + [sl for sl, n in zip(slot_of, lens) for _ in range(n)] + cu + starts + slot_of,
                              dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        ids, positions, token_slot = packed[:T].long(), packed[T:2 * T], packed[2 * T:3 * T]
        B = len(entries)
        cu_t, start_t = packed[3 * T:3 * T + B + 1], packed[3 * T + B + 1:3 * T + 2 * B + 1]
        batch_mapping = packed[3 * T + 2 * B + 1:]
        set_context(is_prefill=max(lens) > 1, cu_seqlens_q=cu_t, cu_seqlens_k=cu_t, max_seqlen_q=max(lens),
                    max_seqlen_k=max(st + n for st, n in zip(starts, lens)), batch_mapping=batch_mapping,
                    positions_i32=positions, token_slot=token_slot, seq_start=start_t)
        hidden = self.model(ids, positions.long())
        row_t = None if rows is None else torch.tensor(list(rows), dtype=torch.int64, device=dev)
        logits = self.model.compute_logits(hidden, row_t)
        reset_context()
        for (s, _), n in zip(entries, lens):
            s.num_computed_tokens += n
        self.stats["steps"] += 1
        self.stats["prefill_tokens"] += sum(n for n in lens if n > 1)
        if temperatures is not None:
            return self.sampler(logits, torch.tensor(list(temperatures), dtype=torch.float32, device=dev))
        return logits

    def _graph_decode_step(self, entries, starts, rows, temperatures=None) -> torch.Tensor:
        """A step of single tokens as a CUDA-graph replay (one graph per padded batch size; padding rows sit on the
        reserved slot, store nothing and attend to nothing).  The graph holds the whole forward pass, the logits of
        every row and the sampler on them; ids, positions, slots and temperatures are copied into its static buffer
        before the replay.  Returns logits rows, or the sampled tokens when temperatures are given."""
        dev = self.device
        B = len(entries)
        bs = _pad_batch(B)
        g = self._step_graphs.get(bs)
        if g is None:
            st = {"packed": torch.zeros(4 * bs, dtype=torch.int32, device=dev)}   # ids, positions, slots, temperatures
            st["packed"][2 * bs:3 * bs] = RESERVED_BATCH

            def forward():
                pk = st["packed"]
                ids, pos, slots = pk[:bs].long(), pk[bs:2 * bs], pk[2 * bs:3 * bs]
                # max_seqlen_k: the replay serves any context length, so the key splits are sized for the longest
                set_context(is_prefill=False, batch_mapping=slots, positions_i32=pos, token_slot=slots,
                            max_seqlen_q=1, max_seqlen_k=self.config.max_model_len)
                hidden = self.model(ids, pos.long())
                # every row's logits: the model's own head function when it has one (a cap on the logits, say)
                head = getattr(self.model, "compute_all_logits", self.model.lm_head)
                out = head(hidden)
                reset_context()
                return out, self.sampler(out, pk[3 * bs:].view(torch.float32))

            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                forward()                      # warm-up on the reserved slot: workspaces, library handles
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    st["logits"], st["tokens"] = forward()
            torch.cuda.current_stream().wait_stream(side)
            g = self._step_graphs[bs] = (graph, st)
        graph, st = g
        pad = bs - B
        slot_of = [self.kv.seq_id_to_batch[s.seq_id] for s, _ in entries]
        host = torch.tensor([toks[0] for _, toks in entries] + [0] * pad + list(starts) + [0] * pad
                            + slot_of + [RESERVED_BATCH] * pad, dtype=torch.int32)
        if temperatures is not None:   # the fourth quarter of the buffer holds fp32 bit patterns
            temps = torch.tensor(list(temperatures) + [0.0] * pad, dtype=torch.float32).view(torch.int32)
            host = torch.cat([host, temps])
        st["packed"][:host.numel()].copy_(host.pin_memory(), non_blocking=True)
        graph.replay()
        if temperatures is not None:
            return st["tokens"][:B]
        pick = list(range(B)) if rows is None else list(rows)
        return st["logits"].index_select(0, torch.tensor(pick, dtype=torch.int64, device=dev))

    def release(self, seqs: Seq[Sequence]) -> None:
        """Give back the slots and pages of finished sequences."""
        for s in seqs:
            self._room.pop(s.seq_id, None)
        self.kv.free_sequences([s.seq_id for s in seqs])

    @torch.no_grad()
    def _generate_stepwise(self, seqs: List[Sequence]) -> None:
        """Continuous batching for models with `mixed_steps`: each step carries one token of every decoding
        sequence plus portions of waiting prompts up to the step's token budget; a sequence is admitted when a slot
        and pages for its prompt and its completion are free, and gives them back when it finishes."""
        waiting, running = deque(seqs), []
        budget = max(int(self.max_batched_tokens), 1)
        while waiting or running:
            while waiting and len(running) < self.config.max_num_seqs and self.kv.num_free_batches > 0:
                s = waiting[0]
                n = s.num_prompt_tokens
                assert 0 < n <= self.config.max_model_len, "prompt longer than max_model_len"
                need = min(n + s.sampling_params.max_new_tokens, self.config.max_model_len)
                if need > self.kv.num_free_tokens:
                    break
                assert self._make_room(s, need)
                s.status = SequenceStatus.RUNNING
                running.append(waiting.popleft())
            if not running:
                raise KVCacheExhausted(f"sequence {waiting[0].seq_id} does not fit an empty cache")
            entries, left = [], budget
            for s in running:      # decoding sequences first: they take one token each
                if s.num_computed_tokens >= s.num_prompt_tokens:
                    entries.append((s, [s.completion_token_ids[-1]]))
                    left -= 1
            for s in running:
                done = s.num_computed_tokens
                if done < s.num_prompt_tokens and left > 0:
                    n = min(s.num_prompt_tokens - done, left)
                    entries.append((s, s.prompt_token_ids[done:done + n]))
                    left -= n
            # every entry gets a token sampled after its last position (in the graph for single-token steps); the
            # ones of prompts that are not finished yet are dropped
            toks = self.run_step(entries, temperatures=[s.sampling_params.temperature for s, _ in entries]).tolist()
            for (s, _), t in zip(entries, toks):
                if s.num_computed_tokens >= s.num_prompt_tokens:
                    self._accept(s, t)
            self.stats["decode_steps"] += 1
            finished = [s for s in running if s.status is SequenceStatus.FINISHED]
            if finished:
                self.release(finished)
                running = [s for s in running if s.status is not SequenceStatus.FINISHED]

    # ----------------------------------------------------------------- generate
    @torch.no_grad()
    def generate(self, seqs: List[Sequence], params: BatchCompressionParams) -> None:
        """Fill `completion_token_ids` of every sequence (reference: core/model_runner.py:230-338)."""
        if self.mixed_steps:
            return self._generate_stepwise(seqs)
        wave = self.config.max_num_seqs
        for w0 in range(0, len(seqs), wave):
            chunk = seqs[w0:w0 + wave]
            for batch in self._prefill_batches(chunk):
                logits = self.run_prefill(batch, params)
                temps = torch.tensor([s.sampling_params.temperature for s in batch], device=self.device)
                first = self.sampler(logits, temps).tolist()
                for s, t in zip(batch, first):
                    s.status = SequenceStatus.RUNNING
                    self._accept(s, t)
            self.run_decode_loop(chunk)
            self.kv.free_sequences([s.seq_id for s in chunk])
