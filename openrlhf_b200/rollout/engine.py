"""Rollout engine: paged KV cache, slot-based continuous batching, CUDA-graph decode loop, prefix sharing for the
n samples of a prompt, sleep / wake and in-place weight updates.

This is the component that takes the place of vLLM in the reference (openrlhf/trainer/ray/vllm_engine.py:63-208 wraps
``vllm.AsyncLLMEngine``; sampling parameters come from openrlhf/trainer/ppo_utils/samples_generator.py:203-211).
Token-in / token-out API: ``generate(prompt_token_ids, sampling_params)`` returns objects with
``.outputs[i].token_ids / .logprobs / .finish_reason`` like the engine the reference's agent executors talk to.

Execution model: every request owns one row ("slot") of a set of static device tensors for its lifetime; one decode
step for all rows is captured once per batch-size bucket as a CUDA graph (embedding -> [RMSNorm, qkv GEMM,
RoPE+KV-write, paged tcgen05 attention, o-proj GEMM(+residual), RMSNorm, gate_up GEMM, SwiGLU, down GEMM(+residual)]
x L -> RMSNorm -> lm_head GEMM -> sampler -> advance) and replayed per token; the host only intervenes every few steps
to hand out KV pages and retire finished rows.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
from dataclasses import dataclass, field

import torch

from ..models.config import ModelConfig
from ..models.transformer import TransformerLM
from ..ops import _lib
from ..ops import functional as F
from ..ops.attention import PAGE, paged_decode, rope_kvwrite
from ..ops.gemm import gemm, gemm_swiglu, swiglu_fusable
from ..ops.sampling import sample
from .block_manager import BlockManager


import os as _os

_DEBUG = _os.environ.get("OPENRLHF_B200_DEBUG", "0") == "1"


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    max_tokens: int | None = 16
    min_tokens: int = 0
    n: int = 1
    logprobs: int | None = None
    ignore_eos: bool = False
    stop_token_ids: list | None = None
    seed: int | None = None
    skip_special_tokens: bool = False
    include_stop_str_in_output: bool = False


@dataclass
class Logprob:
    logprob: float
    rank: int | None = None
    decoded_token: str | None = None


@dataclass
class CompletionOutput:
    index: int
    token_ids: list
    logprobs: list | None          # [{token_id: Logprob}] per generated token when requested
    finish_reason: str
    text: str = ""
    cumulative_logprob: float = 0.0
    logprob_values: list | None = None   # plain floats, always filled


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list
    outputs: list = field(default_factory=list)
    finished: bool = True


@dataclass
class _Row:
    request_id: int
    sample_index: int
    prompt_len: int              # tokens in front of the first token this row still has to generate (prompt, plus the
                                 # tokens generated before a preemption)
    max_tokens: int              # total tokens the sample may generate
    pages: list
    gen: int = 0                 # tokens generated so far as far as the host knows (upper bound for finished rows)
    base: int = 0                # tokens generated before this row was (re)admitted: restored after a preemption
    order: int = 0               # admission order (the newest rows are preempted first)
    prefilled: int = -1          # chunked prefill: context tokens whose KV is in the cache; -1 once decoding


@dataclass
class _Pending:
    """A queued request, or one preempted sample waiting to be recomputed (`done_*` hold what it had generated)."""
    request_id: object
    prompt: list
    sp: "SamplingParams"
    mm: dict | None = None
    sample_index: int | None = None       # set for a preempted sample (one row); None: a fresh request with sp.n rows
    done_tokens: list = field(default_factory=list)
    done_logprobs: list = field(default_factory=list)


class RolloutEngine:
    def __init__(self, model: TransformerLM, max_num_seqs: int = 256, max_model_len: int = 4096,
                 num_pages: int | None = None, gpu_memory_utilization: float = 0.5, seed: int = 0,
                 eos_token_id: int | None = None, use_cuda_graph: bool = True, check_interval: int = 16, tp=None,
                 quantization: str | None = None, enable_prefix_caching: bool = False,
                 max_prefill_tokens: int = 16384, decode_pdl: bool = False):
        assert model.cfg.head_dim == 128 or not model.flat.is_cuda, \
            "the decode attention kernel is specialised for head_dim 128"
        assert quantization in (None, "fp8"), "rollout quantisation: None or 'fp8' (per-tensor e4m3)"
        self.model = model
        # fp8 decode: the projection weights are kept as e4m3 copies with one scale per matrix (re-quantised after
        # every weight update), activations are quantised per call; halves the weight bytes a decode step streams.
        # Prefill, attention, norms and the lm_head stay bf16.
        self.quantization = quantization
        # fused decode layers launched as a programmatic-dependent-launch chain; off by default: on the decode loops
        # measured (Qwen2.5-1.5B at batch 128, Qwen2.5-7B at batch 64) it changes the step time by less than 1 %
        self.decode_pdl = decode_pdl
        self.fp8: dict = {}
        self.tp = tp          # rollout.tp_engine.TPDecode: `model` then holds this rank's tensor-parallel shard
        self.cfg: ModelConfig = model.cfg
        self.device = model.flat.device
        # CPU tensors run the PyTorch restatements of every kernel (scheduler, launcher and agent tests without a GPU)
        self.on_gpu = self.device.type == "cuda"
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_pages = (max_model_len + PAGE - 1) // PAGE
        self.seed = seed
        self.eos = self.cfg.eos_token_id if eos_token_id is None else eos_token_id
        self.use_cuda_graph = use_cuda_graph and self.on_gpu
        self.check_interval = check_interval
        cfg = self.cfg
        bytes_per_page = 2 * cfg.num_hidden_layers * PAGE * cfg.kv_size * 2
        if num_pages is None and not self.on_gpu:
            num_pages = max(8, min(max_num_seqs * self.max_pages + 1, 2048))
        if num_pages is None:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(total * gpu_memory_utilization) - (total - free)
            num_pages = max(8, min(budget // bytes_per_page, max_num_seqs * self.max_pages + 1))
        self.num_pages = int(num_pages)
        self.blocks = BlockManager(self.num_pages)
        self.dummy_page = self.blocks.alloc()  # page 0 backs inactive rows
        self.kv = None
        self.arena = None
        self._alloc_kv()
        B = max_num_seqs
        dev = self.device
        self.tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        # vision-language models: rotary position of a generated token = token index + the prompt's M-RoPE offset
        self.mrope = cfg.is_vlm
        self.rope_delta = torch.zeros(B, dtype=torch.int32, device=dev)
        self.rope_pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.seq_lens = torch.ones(B, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(B, dtype=torch.int32, device=dev)
        self.block_table = torch.full((B, self.max_pages), self.dummy_page, dtype=torch.int32, device=dev)
        self.block_table_host = torch.full((B, self.max_pages), self.dummy_page, dtype=torch.int32)
        if self.on_gpu:
            self.block_table_host = self.block_table_host.pin_memory()
        self.active = torch.zeros(B, dtype=torch.int32, device=dev)
        self.gen_count = torch.zeros(B, dtype=torch.int32, device=dev)
        self.max_tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.min_tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.ignore_eos = torch.zeros(B, dtype=torch.bool, device=dev)
        self.temperature = torch.ones(B, dtype=torch.float32, device=dev)
        # nucleus settings are per request (one value per row), like the sampling parameters of the reference's engine
        self.top_k_rows = torch.full((B,), -1, dtype=torch.int32, device=dev)
        self.top_p_rows = torch.ones(B, dtype=torch.float32, device=dev)
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=dev)
        self.max_new_cap = max_model_len
        self.out_tokens = torch.zeros(B, self.max_new_cap, dtype=torch.int64, device=dev)
        self.out_logprobs = torch.zeros(B, self.max_new_cap, dtype=torch.float32, device=dev)
        self.q_buf = torch.empty(B, cfg.num_attention_heads, cfg.head_dim, dtype=model.flat.dtype, device=dev)
        self.attn_buf = torch.empty_like(self.q_buf)
        self.next_tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.next_lp = torch.zeros(B, dtype=torch.float32, device=dev)
        self.rows: list[_Row | None] = [None] * B
        from collections import deque

        self.waiting = deque()
        self._prefilling: list = []             # admitted requests whose context is not fully prefilled yet
        self._table_dirty = False
        self._stale_rows: list = []
        self._req: dict = {}
        self._batch_counter = 0
        self.graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
        self.graph_launches: dict[tuple, int] = {}
        self.sleeping = False
        self.paused = False
        self.decode_steps = 0
        self._quiet_bursts = 0     # consecutive decode bursts in which no row finished and nothing was waiting
        # scheduler state: admission order, chunked-prefill budget, prefix cache, preemption counters
        self.max_prefill_tokens = max(int(max_prefill_tokens), PAGE)
        self._order = 0
        self.enable_prefix_caching = bool(enable_prefix_caching)
        from collections import OrderedDict

        self._cache: "OrderedDict[int, int]" = OrderedDict()   # chain hash of a full page of tokens -> page (LRU order)
        self._cache_hash: dict[int, int] = {}                  # page -> its hash
        self._cache_users: dict[int, int] = {}                 # page -> live rows reading it
        self.stats = {"preemptions": 0, "prefix_hit_tokens": 0, "prefill_tokens": 0, "prefill_chunks": 0}
        if self.on_gpu:
            _lib.status_word(self.device)
        self.model.rope(self.device)

    # ------------------------------------------------------------------ memory
    def _alloc_kv(self):
        """KV cache [layers, 2, pages*128, kv_heads, 128] inside a VMM arena: its address survives sleep / wake."""
        cfg = self.cfg
        shape = (cfg.num_hidden_layers, 2, self.num_pages * PAGE, cfg.num_key_value_heads, cfg.head_dim)
        if not self.on_gpu:
            self.kv = torch.zeros(*shape, dtype=self.model.flat.dtype, device=self.device)
            return
        if getattr(self, "arena", None) is None:
            try:
                from .block_manager import VmmArena

                nbytes = 2
                for d in shape:
                    nbytes *= d
                self.arena = VmmArena(nbytes, self.device)
            except Exception:  # noqa: BLE001  (driver without VMM support: plain allocation, graphs dropped on sleep)
                self.arena = None
        if self.arena is not None:
            if not self.arena.mapped:
                self.arena.map()
            self.kv = self.arena.tensor(torch.bfloat16, shape)
            self.kv.zero_()       # stale V rows are multiplied by zero probabilities: they must be finite
        else:
            self.kv = torch.zeros(*shape, dtype=torch.bfloat16, device=self.device)

    def sleep(self, level: int = 1):
        """Release the physical memory of the KV cache. Weights stay resident: trainer and rollout share them on this
        GPU. With the VMM arena the cache keeps its address, so captured decode graphs stay valid across sleep / wake
        (counterpart of vLLM sleep mode as used at openrlhf/trainer/ray/vllm_engine.py:138-153)."""
        if self.sleeping:
            return
        if self.arena is not None:
            self.arena.unmap()
        else:
            self.graphs.clear()
            self.kv = None
            if self.on_gpu:
                torch.cuda.empty_cache()
        self.sleeping = True

    def wake_up(self, tags=None):
        if tags is not None and "kv_cache" not in tags:
            return  # weights are always resident
        if self.sleeping:
            self._alloc_kv()
        self.sleeping = False

    def reset_prefix_cache(self):
        """Forget every cached prefix (their KV was computed with weights that have been replaced). Pages that live
        rows still read stay allocated until those rows finish."""
        for page in list(self._cache_hash):
            self.blocks.free(page)                 # the cache's own reference
        self._cache.clear()
        self._cache_hash.clear()
        self._cache_users.clear()
        return True

    def pause_generation(self):
        self.paused = True

    def resume_generation(self):
        self.paused = False

    def get_num_unfinished_requests(self) -> int:
        return sum(r is not None for r in self.rows) + len(self.waiting)

    @torch.no_grad()
    def update_weights(self, flat_src: torch.Tensor):
        """Copy a new set of weights (same flat layout) into the engine's buffer; a no-op when they alias."""
        if self._cache_hash:
            self.reset_prefix_cache()
        if self.tp is not None:
            if flat_src is None:
                self.tp.refresh(self.model.flat)               # from the configured source (ZeRO-3 slices, ...)
            else:
                self.tp.load_shard(flat_src, self.model.flat)  # one planned copy kernel: full layout -> this TP shard
            return
        if flat_src.data_ptr() != self.model.flat.data_ptr():
            n = min(flat_src.numel(), self.model.flat.numel())      # buffers may differ in their shard padding
            self.model.flat[:n].copy_(flat_src[:n], non_blocking=True)
        if self.quantization == "fp8":
            self._refresh_fp8()

    @torch.no_grad()
    def _refresh_fp8(self):
        from ..ops.fp8 import Fp8Linear

        cfg, m = self.cfg, self.model
        assert cfg.num_experts == 0 and m.lora is None and self.tp is None, \
            "fp8 rollout covers dense models without adapters or tensor parallelism"
        for i in range(cfg.num_hidden_layers):
            pre = f"layers.{i}."
            for t in ("qkv", "o", "gate_up", "down"):
                self.fp8[(i, t)] = Fp8Linear(m.p(pre + t + ".weight"), m._params.get(pre + t + ".bias"))

    # ------------------------------------------------------------------ model execution
    @torch.no_grad()
    def _prefill(self, items: list, mms: list | None = None):
        """Run one prefill pass. items: list of (tokens, start, row) where `tokens` is the whole context of the row so
        far (prompt, plus generated tokens of a preempted sample), `start` the number of leading tokens whose KV already
        sits in the row's pages (prefix-cache hit or earlier chunks) and the rest, tokens[start:], is computed now and
        written to the pages of `row`. Returns the logits [len(items), V] at the last position of every item.
        mms: per item None or {"pixel_values", "image_grid_thw"} (only with start == 0); sets the rotary offsets."""
        cfg, m = self.cfg, self.model
        dev = self.device
        n_items = len(items)
        new_lens = [len(t) - s0 for t, s0, _ in items]
        starts = [s0 for _, s0, _ in items]
        ids = torch.tensor([x for t, s0, _ in items for x in t[s0:]], dtype=torch.int64, device=dev)
        pos = torch.cat([torch.arange(s0, s0 + n, dtype=torch.int32) for s0, n in zip(starts, new_lens)]).to(dev)
        cu_new = [0]
        for n in new_lens:
            cu_new.append(cu_new[-1] + n)
        cu = torch.tensor(cu_new, dtype=torch.int32, device=dev)

        def slots_of(row, a, b):
            pages = self.rows[row].pages
            return [pages[t // PAGE] * PAGE + t % PAGE for t in range(a, b)]

        slots = torch.tensor([x for (t, s0, row) in items for x in slots_of(row, s0, len(t))], dtype=torch.int64,
                             device=dev)
        with_prefix = any(starts)
        if with_prefix:
            # rows of the full (prefix + new) stream: where each sequence's cached keys live, and where the new ones go
            cu_all = [0]
            for t, _, _ in items:
                cu_all.append(cu_all[-1] + len(t))
            pre_slots = torch.tensor([x for (t, s0, row) in items for x in slots_of(row, 0, s0)], dtype=torch.int64,
                                     device=dev)
            pre_rows = torch.cat([torch.arange(cu_all[i], cu_all[i] + starts[i]) for i in range(n_items)]).to(dev)
            new_rows = torch.cat([torch.arange(cu_all[i] + starts[i], cu_all[i + 1]) for i in range(n_items)]).to(dev)
            scale = 1.0 / math.sqrt(cfg.head_dim)

        def attn_fn(i, q, k, v):
            self.kv[i, 0].index_copy_(0, slots, k)
            self.kv[i, 1].index_copy_(0, slots, v)
            if not with_prefix:
                return F.attention_varlen(q, k, v, cu, max(new_lens))
            from ..ops.attention import attention_with_prefix

            k_all = torch.empty(cu_all[-1], k.shape[1], k.shape[2], dtype=k.dtype, device=dev)
            v_all = torch.empty_like(k_all)
            k_all.index_copy_(0, pre_rows, self.kv[i, 0].index_select(0, pre_slots))
            v_all.index_copy_(0, pre_rows, self.kv[i, 1].index_select(0, pre_slots))
            k_all.index_copy_(0, new_rows, k)
            v_all.index_copy_(0, new_rows, v)
            return attention_with_prefix(q, k_all, v_all, cu_all, starts, scale)

        was_training = m.training
        m.eval()
        embeds = None
        if self.mrope:
            deltas = [0] * n_items
            if mms and any(mms):
                from ..models.vision import mrope_positions

                assert not with_prefix, "image prompts are prefilled in one piece"
                pv = torch.cat([mm["pixel_values"] for mm in mms if mm]).to(dev)
                thw = torch.cat([torch.as_tensor(mm["image_grid_thw"]).view(-1, 3) for mm in mms if mm])
                embeds, pos = m.multimodal_inputs(ids, cu_new, pv, thw)
                merge = cfg.vision_config().spatial_merge_size
                for k_, ((t, _, _), mm) in enumerate(zip(items, mms)):
                    if mm:
                        grids = [tuple(g) for g in torch.as_tensor(mm["image_grid_thw"]).view(-1, 3).tolist()]
                        deltas[k_] = mrope_positions(t, grids, cfg.image_token_id, merge, cfg.video_token_id)[1]
            for d, (_, _, row) in zip(deltas, items):
                self.rope_delta[row] = d
        # ranks prefill independently of each other: expert-parallel dispatch (a collective of the training passes) is
        # off here, every rank runs all experts of its own copy of the weights
        ep_saved, m.ep = m.ep, None
        try:
            h, _ = m(ids, pos, cu, max(new_lens), attn_fn=attn_fn, inputs_embeds=embeds)
        finally:
            m.ep = ep_saved
        m.train(was_training)
        last = (cu[1:] - 1).long()
        self.stats["prefill_tokens"] += int(cu_new[-1])
        self.stats["prefill_chunks"] += 1
        return F.linear(h[last].contiguous(), m.lm_head_weight())

    def _decode_step(self, B: int):
        """One token for rows [0, B). Pure device work on static buffers: safe to capture in a CUDA graph."""
        cfg, m = self.cfg, self.model
        fused = (not cfg.qk_norm and cfg.num_experts == 0 and m.lora is None and self.quantization is None
                 and self.on_gpu)
        if self.quantization == "fp8" and not self.fp8:
            self._refresh_fp8()
        if self.mrope:
            torch.add(self.pos[:B], self.rope_delta[:B], out=self.rope_pos[:B])
        if fused:
            # launch- and prologue-bound chain of small kernels over static weights: programmatic dependent launch
            with (_lib.decode_chain() if self.decode_pdl else contextlib.nullcontext()):
                logits = self._decode_layers_fused(B)
        else:
            logits = self._decode_layers_generic(B)
        sample(logits, temperature=self.temperature[:B], top_k=self.top_k_rows[:B], top_p=self.top_p_rows[:B], seed=self.seed,
               step=self.step_counter, out_tokens=self.next_tok[:B], out_logprobs=self.next_lp[:B],
               active=self.active[:B])
        self._advance(B)

    def _decode_layers_fused(self, B: int):
        """Dense decoder layers in 8 launches each: every split-K projection leaves fp32 slabs in the workspace and the
        kernel that follows finishes the reduction together with its own work (bias + RoPE + KV write after qkv,
        residual + RMSNorm after o_proj and down_proj)."""
        cfg, m = self.cfg, self.model
        L = _lib.lib()
        Hq, Hkv, H = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size
        scale = 1.0 / math.sqrt(cfg.head_dim)
        table = m.rope(self.device)
        tok, pos, slots = self.tok[:B], (self.rope_pos if self.mrope else self.pos)[:B], self.slots[:B]
        bt, sl = self.block_table[:B], self.seq_lens[:B]
        q_buf, attn_buf = self.q_buf[:B], self.attn_buf[:B]
        st = _lib.stream_ptr
        i32, f32 = ctypes.c_int, ctypes.c_float

        tp = self.tp

        def reduce_norm(ws, splits, residual, w, which=0):
            h = torch.empty(B, H, dtype=torch.bfloat16, device=self.device)
            x = torch.empty_like(h)
            if tp is not None:
                # row-parallel projection: all ranks' slabs are summed here (the all-reduce rides on the reduction)
                tp.barrier()
                rc = L.b200_tp_reduce_rmsnorm(tp.ws_ptrs[which], i32(tp.size), i32(splits), _lib.ptr(residual),
                                              _lib.ptr(w), _lib.ptr(h), _lib.ptr(x), i32(B), i32(H),
                                              f32(cfg.rms_norm_eps), st())
                _lib.check_rc(rc, "tp_reduce_rmsnorm")
                return h, x
            rc = L.b200_splitk_reduce_rmsnorm(_lib.ptr(ws), i32(splits), _lib.ptr(residual), _lib.ptr(w), _lib.ptr(h),
                                              _lib.ptr(x), i32(B), i32(H), f32(cfg.rms_norm_eps), st())
            _lib.check_rc(rc, "splitk_reduce_rmsnorm")
            return h, x

        h = F.embedding(tok, m.p("embed.weight"))
        x = F.rmsnorm(h, m.p("layers.0.norm1.weight"), cfg.rms_norm_eps)
        nl = cfg.num_hidden_layers
        for i in range(nl):
            pre = f"layers.{i}."
            ws, s = gemm_to_workspace(x, m.p(pre + "qkv.weight"))
            rc = L.b200_rope_kvwrite_splitk(_lib.ptr(ws), i32(s), _lib.ptr(m._params.get(pre + "qkv.bias")),
                                            _lib.ptr(pos), _lib.ptr(slots), _lib.ptr(table), _lib.ptr(q_buf),
                                            _lib.ptr(self.kv[i, 0]), _lib.ptr(self.kv[i, 1]), i32(B), i32(Hq), i32(Hkv),
                                            i32(table.shape[0]), st())
            _lib.check_rc(rc, "rope_kvwrite_splitk")
            paged_decode(q_buf, self.kv[i, 0], self.kv[i, 1], bt, sl, scale, out=attn_buf)
            ws, s = gemm_to_workspace(attn_buf.view(B, Hq * 128), m.p(pre + "o.weight"),
                                      tp.ws[0] if tp is not None else None)
            h, x = reduce_norm(ws, s, h, m.p(pre + "norm2.weight"), 0)
            wgu = m.p(pre + "gate_up.weight")
            if swiglu_fusable(wgu.shape[0] // 2):
                a, _ = gemm_swiglu(x, wgu, bn=128)          # SwiGLU in the GEMM epilogue: one launch less per layer
            else:
                a = F.swiglu(gemm(x, wgu, bn=128))
            ws, s = gemm_to_workspace(a, m.p(pre + "down.weight"), tp.ws[1] if tp is not None else None)
            nxt = m.p(f"layers.{i + 1}.norm1.weight") if i + 1 < nl else m.p("norm.weight")
            h, x = reduce_norm(ws, s, h, nxt, 1)
        return gemm(x, m.lm_head_weight())

    def _decode_layers_generic(self, B: int):
        cfg, m = self.cfg, self.model
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        scale = 1.0 / math.sqrt(cfg.head_dim)
        table = m.rope(self.device)
        tok, pos, slots = self.tok[:B], (self.rope_pos if self.mrope else self.pos)[:B], self.slots[:B]
        bt, sl = self.block_table[:B], self.seq_lens[:B]
        q_buf, attn_buf = self.q_buf[:B], self.attn_buf[:B]
        h = F.embedding(tok, m.p("embed.weight"))
        for i in range(cfg.num_hidden_layers):
            pre = f"layers.{i}."
            x = F.rmsnorm(h, m.p(pre + "norm1.weight"), cfg.rms_norm_eps)
            if self.quantization == "fp8":
                qkv = self.fp8[(i, "qkv")](x)
            else:
                qkv = m._lin(i, "qkv", x, m._params.get(pre + "qkv.bias")) if m.lora is not None else \
                    decode_gemm(x, m.p(pre + "qkv.weight"), m._params.get(pre + "qkv.bias"))
            if cfg.qk_norm:
                T = qkv.shape[0]
                qk = qkv[:, : (Hq + Hkv) * 128].reshape(T, Hq + Hkv, 128)
                qn = F.rmsnorm(qk[:, :Hq].reshape(-1, 128), m.p(pre + "q_norm.weight"), cfg.rms_norm_eps).view(T, -1)
                kn = F.rmsnorm(qk[:, Hq:].reshape(-1, 128), m.p(pre + "k_norm.weight"), cfg.rms_norm_eps).view(T, -1)
                qkv = torch.cat([qn, kn, qkv[:, (Hq + Hkv) * 128:]], dim=1)
            rope_kvwrite(qkv, pos, slots, table, q_buf, self.kv[i, 0], self.kv[i, 1], Hq, Hkv)
            paged_decode(q_buf, self.kv[i, 0], self.kv[i, 1], bt, sl, scale, out=attn_buf)
            ao = attn_buf.view(B, Hq * cfg.head_dim)
            if self.tp is not None:
                # row-parallel shard outside the fused path (qk-norm / MoE models, CPU ranks): partial product, sum
                # over the tensor-parallel group, residual once
                h = h + self.tp.all_reduce(decode_gemm(ao, m.p(pre + "o.weight")))
            elif self.quantization == "fp8":
                h = self.fp8[(i, "o")](ao, residual=h)
            else:
                h = m._lin(i, "o", ao, None, h) if m.lora is not None else decode_gemm(ao, m.p(pre + "o.weight"), None, h)
            x = F.rmsnorm(h, m.p(pre + "norm2.weight"), cfg.rms_norm_eps)
            if cfg.is_moe_layer(i):
                from ..models.moe import moe_forward

                y, _ = moe_forward(x, m.p(pre + "router.weight"), m.p(pre + "experts.gate_up"),
                                   m.p(pre + "experts.down"), cfg.num_experts_per_tok, cfg.norm_topk_prob)
                h = h + y
            elif self.quantization == "fp8":
                h = self.fp8[(i, "down")](F.swiglu(self.fp8[(i, "gate_up")](x)), residual=h)
            elif m.lora is not None:
                h = m._lin(i, "down", F.swiglu(m._lin(i, "gate_up", x)), None, h)
            elif self.tp is not None:
                a = F.swiglu(decode_gemm(x, m.p(pre + "gate_up.weight")))
                h = h + self.tp.all_reduce(decode_gemm(a, m.p(pre + "down.weight")))
            else:
                gu = decode_gemm(x, m.p(pre + "gate_up.weight"))
                a = F.swiglu(gu)
                h = decode_gemm(a, m.p(pre + "down.weight"), None, h)
        x = F.rmsnorm(h, m.p("norm.weight"), cfg.rms_norm_eps)
        return F.linear(x, m.lm_head_weight())

    def _advance(self, B: int):
        """Per-step bookkeeping (append token / log-prob, stop conditions, next position and KV slot): one kernel."""
        if self.tok.is_cuda:
            import ctypes

            rc = _lib.lib().b200_decode_advance(
                ctypes.c_int(B), _lib.ptr(self.next_tok), _lib.ptr(self.next_lp), _lib.ptr(self.tok), _lib.ptr(self.pos),
                _lib.ptr(self.seq_lens), _lib.ptr(self.slots), _lib.ptr(self.active), _lib.ptr(self.gen_count),
                _lib.ptr(self.out_tokens), _lib.ptr(self.out_logprobs), ctypes.c_int(self.max_new_cap),
                _lib.ptr(self.min_tok), _lib.ptr(self.max_tok), _lib.ptr(self.ignore_eos), ctypes.c_longlong(self.eos),
                _lib.ptr(self.block_table), ctypes.c_int(self.max_pages), ctypes.c_int(PAGE),
                _lib.ptr(self.step_counter), _lib.stream_ptr())
            _lib.check_rc(rc, "decode_advance")
            return
        act = self.active[:B].bool()
        g = self.gen_count[:B].long().clamp_max(self.max_new_cap - 1)
        rows = torch.arange(B, device=self.device)
        nt = torch.where(act, self.next_tok[:B], self.tok[:B])
        self.out_tokens[rows, g] = torch.where(act, nt, self.out_tokens[rows, g])
        self.out_logprobs[rows, g] = torch.where(act, self.next_lp[:B], self.out_logprobs[rows, g])
        inc = act.int()
        self.gen_count[:B] += inc
        gc = self.gen_count[:B]
        hit_eos = (nt == self.eos) & ~self.ignore_eos[:B] & (gc >= self.min_tok[:B])
        done = act & (hit_eos | (gc >= self.max_tok[:B]))
        still = act & ~done
        self.tok[:B] = nt
        self.pos[:B] += still.int()
        self.seq_lens[:B] += still.int()
        self.active[:B] = still.int()
        p = self.pos[:B].long()
        page = self.block_table[:B].gather(1, (p // PAGE).clamp_max(self.max_pages - 1)[:, None]).squeeze(1)
        self.slots[:B] = (page * PAGE + (p % PAGE).int()).int()
        self.step_counter += 1

    def _run_decode(self, B: int):
        if not self.use_cuda_graph:
            self._decode_step(B)
            return
        key = (B,)
        g = self.graphs.get(key)
        if g is None:
            # warm up outside capture (lazy library state, status word, rope table), then capture
            saved = self._snapshot_state(B)
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_step(B)
            torch.cuda.current_stream().wait_stream(s)
            self._restore_state(saved, B)
            g = torch.cuda.CUDAGraph()
            before = _lib.LAUNCHES
            with torch.cuda.graph(g):
                self._decode_step(B)
            self.graph_launches[key] = _lib.LAUNCHES - before
            self._restore_state(saved, B)
            self.graphs[key] = g
        g.replay()
        _lib.count_launches(self.graph_launches[key])

    def _state_tensors(self):
        return [self.tok, self.pos, self.seq_lens, self.slots, self.active, self.gen_count, self.step_counter,
                self.out_tokens, self.out_logprobs]

    def _snapshot_state(self, B):
        return [t.clone() for t in self._state_tensors()]

    def _restore_state(self, saved, B):
        for t, s in zip(self._state_tensors(), saved):
            t.copy_(s)

    # ------------------------------------------------------------------ scheduling: pages
    def _bucket(self, n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return min(b, self.max_num_seqs)

    def _evictable(self) -> int:
        return sum(1 for p, u in self._cache_users.items() if u == 0)

    def _free_pages(self) -> int:
        """Pages obtainable right now: free ones plus cached prefixes no live row is reading."""
        return self.blocks.num_free() + self._evictable()

    def _alloc_page(self) -> int:
        if self.blocks.num_free() == 0:
            for h, page in self._cache.items():          # least recently used first
                if self._cache_users.get(page, 0) == 0:
                    del self._cache[h]
                    del self._cache_hash[page]
                    del self._cache_users[page]
                    self.blocks.free(page)
                    break
        return self.blocks.alloc()

    def _sync_block_table(self):
        """Host block table -> device. Rows that are still being prefilled show the dummy page on the device: the
        decode kernels run over all rows of a bucket, and an inactive row writes its (meaningless) K/V at whatever
        slot its table row and stale position give - that must never be a page of a live context."""
        self._table_dirty = False
        if self._stale_rows:
            # a released row keeps running in the decode kernels as an inactive row: park its write slot on the dummy
            # page, or its next (meaningless) K/V write would land in a page that now belongs to another context
            idx = torch.tensor(self._stale_rows, dtype=torch.int64, device=self.device)
            self.slots[idx] = self.dummy_page * PAGE
            self.pos[idx] = 0
            self.seq_lens[idx] = 1
            self._stale_rows = []
        hold = [r for _, rows, _ in self._prefilling for r in rows]
        if hold:
            tmp = self.block_table_host.clone()
            tmp[hold] = self.dummy_page
            self.block_table.copy_(tmp)
        else:
            self.block_table.copy_(self.block_table_host, non_blocking=True)

    def _pages_short(self, row: int, upto_pos: int) -> int:
        need = min(upto_pos, self.max_model_len - 1) // PAGE + 1
        return max(0, need - len(self.rows[row].pages))

    def _ensure_pages(self, row: int, upto_pos: int):
        r = self.rows[row]
        need = min(upto_pos, self.max_model_len - 1) // PAGE + 1
        changed = False
        while len(r.pages) < need:
            pg = self._alloc_page()
            r.pages.append(pg)
            self.block_table_host[row, len(r.pages) - 1] = pg
            changed = True
        return changed

    def _release_pages(self, pages: list):
        for pg in pages:
            if pg in self._cache_users:
                self._cache_users[pg] -= 1
            self.blocks.free(pg)

    def _release_row(self, row: int):
        self._release_pages(self.rows[row].pages)
        self.rows[row] = None
        self.block_table_host[row].fill_(self.dummy_page)
        self._table_dirty = True
        self._stale_rows.append(row)

    # ------------------------------------------------------------------ scheduling: prefix cache
    @staticmethod
    def _page_hashes(tokens: list, n_pages: int) -> list:
        """Chain hashes of the first n_pages full pages of a token list (a page's hash covers everything before it)."""
        out, h = [], 0
        for i in range(n_pages):
            h = hash((h, tuple(tokens[i * PAGE:(i + 1) * PAGE])))
            out.append(h)
        return out

    def _cache_lookup(self, tokens: list) -> list:
        """Pages holding the KV of the longest cached prefix of `tokens` (whole pages; at least one token is left to
        compute so that the prefill yields logits)."""
        if not self.enable_prefix_caching:
            return []
        hits = []
        for h in self._page_hashes(tokens, (len(tokens) - 1) // PAGE):
            page = self._cache.get(h)
            if page is None:
                break
            hits.append(page)
        return hits

    def _cache_insert(self, tokens: list, pages: list, n_full: int):
        """Offer the first n_full pages of a row (whose KV is complete) to the cache; it keeps its own reference."""
        if not self.enable_prefix_caching:
            return
        for idx, (h, page) in enumerate(zip(self._page_hashes(tokens, n_full), pages[:n_full])):
            if h in self._cache or page in self._cache_hash:
                if h in self._cache:
                    self._cache.move_to_end(h)
                continue
            self.blocks.share(page)
            self._cache[h] = page
            self._cache_hash[page] = h
            # live rows that read this page (the samples of one request hold their shared pages at the same index)
            self._cache_users[page] = sum(1 for r in self.rows
                                          if r is not None and len(r.pages) > idx and r.pages[idx] == page)

    # ------------------------------------------------------------------ request API (continuous batching)
    def add_request(self, request_id, prompt_token_ids: list[int], sampling_params: SamplingParams,
                    multi_modal_data: dict | None = None) -> None:
        """Queue one request; it is admitted by a later ``step()`` when rows and KV pages are available.
        multi_modal_data: {"pixel_values": [N, patch_dim], "image_grid_thw": [n, 3]} for prompts that contain image
        placeholder tokens (vision-language models), or {"image": [PIL images]} when an image processor is attached
        (``self.image_processor``)."""
        mm = None
        if multi_modal_data:
            assert self.mrope, "this model takes no image inputs"
            mm = self._mm_tensors(multi_modal_data)
        prompt = list(prompt_token_ids)
        if len(prompt) >= self.max_model_len:
            assert mm is None, "a prompt with images exceeds max_model_len (truncation would cut an image)"
            prompt = prompt[-(self.max_model_len - 1):]
        self.waiting.append(_Pending(request_id, prompt, sampling_params, mm))

    image_processor = None

    def _mm_tensors(self, mm: dict) -> dict:
        if "pixel_values" in mm:
            return {"pixel_values": mm["pixel_values"], "image_grid_thw": mm["image_grid_thw"]}
        if self.image_processor is None:
            raise ValueError("multi_modal_data carries images but the engine has no image_processor; pass "
                             "pixel_values / image_grid_thw instead")
        enc = self.image_processor(images=list(mm["image"]), return_tensors="pt")
        return {"pixel_values": enc["pixel_values"], "image_grid_thw": enc["image_grid_thw"]}

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or any(r is not None for r in self.rows)

    def _max_new(self, prompt, sp) -> int:
        m = sp.max_tokens if sp.max_tokens is not None else max(1, self.max_model_len - len(prompt))
        return max(1, min(m, self.max_model_len - len(prompt)))

    # ------------------------------------------------------------------ admission, chunked prefill, preemption
    def _admit(self):
        """Move queued requests into rows while rows and pages last. Pages are taken for the context only (not for
        the tokens still to be generated: decode bursts allocate as they go and preempt when the pool runs dry); one
        page of headroom per live row keeps a freshly admitted request from being preempted straight away."""
        free_rows = [i for i, r in enumerate(self.rows) if r is None]
        admitted = False
        while self.waiting:
            e: _Pending = self.waiting[0]
            n = 1 if e.sample_index is not None else e.sp.n
            tokens = e.prompt + e.done_tokens
            hits = self._cache_lookup(tokens) if e.mm is None else []
            n_full = len(tokens) // PAGE
            own_full = max(0, n_full - len(hits))
            live = sum(r is not None for r in self.rows)
            need = own_full + n                       # shared full pages still to compute + one open page per row
            # hit pages that nobody reads count as obtainable in _free_pages(); pinning them takes them out of it
            pinned = sum(1 for pg in hits if self._cache_users.get(pg, 0) == 0)
            if len(free_rows) < n or self._free_pages() - pinned < need + live + 1:
                if live == 0 and not admitted:
                    self.waiting.popleft()
                    raise RuntimeError("a request does not fit into the KV cache / row budget of the rollout engine")
                break
            self.waiting.popleft()
            for pg in hits:                            # pin before any allocation can evict them
                self._cache_users[pg] += n
                self._cache.move_to_end(self._cache_hash[pg])
            rows = [free_rows.pop(0) for _ in range(n)]
            shared = [self.blocks.share(pg) for pg in hits] + [self._alloc_page() for _ in range(own_full)]
            max_new = self._max_new(e.prompt, e.sp)
            for j, r in enumerate(rows):
                if j > 0:
                    for pg in shared:
                        self.blocks.share(pg)
                self._order += 1
                self.rows[r] = _Row(e.request_id, e.sample_index if e.sample_index is not None else j, len(tokens),
                                    max_new, list(shared), gen=len(e.done_tokens), base=len(e.done_tokens),
                                    order=self._order, prefilled=len(hits) * PAGE)
                self.block_table_host[r].fill_(self.dummy_page)
                for t, pg in enumerate(shared):
                    self.block_table_host[r, t] = pg
                self._ensure_pages(r, len(tokens))
            if e.sample_index is None:
                self._req[e.request_id] = (e.prompt, e.sp, {})
            self.stats["prefix_hit_tokens"] += len(hits) * PAGE
            self._prefilling.append((e, rows, tokens))
            admitted = True

    def _prefill_work(self):
        """Spend up to max_prefill_tokens on the admitted-but-not-yet-decoding requests, oldest first. A context longer
        than the budget is prefilled in chunks over several calls (decode bursts of the live rows run in between);
        once its last chunk is done the rows of the request are started with their first sampled token."""
        budget = self.max_prefill_tokens
        batch, finishing = [], []
        for entry in self._prefilling:
            e, rows, tokens = entry
            lead = self.rows[rows[0]]
            left = len(tokens) - lead.prefilled
            if budget <= 0 or (e.mm is not None and left > budget and batch):
                break
            take = left if e.mm is not None else min(left, budget)     # image prompts are not cut
            upto = lead.prefilled + take
            batch.append((tokens[:upto], lead.prefilled, rows[0]))
            budget -= take
            if upto == len(tokens):
                finishing.append((len(batch) - 1, entry))
            else:
                lead.prefilled = upto
                break                                   # an unfinished context uses up the pass
        if not batch:
            return
        logits = self._prefill(batch, [en[0].mm if (en[0].mm is not None and b[1] == 0) else None
                                       for en, b in zip(self._prefilling, batch)])
        if finishing:
            done = {id(en) for _, en in finishing}
            self._prefilling = [en for en in self._prefilling if id(en) not in done]
            self._sync_block_table()                   # the finished rows' pages become visible to the decode kernels
            self._start_rows(logits[[k for k, _ in finishing]], [en for _, en in finishing])
        else:
            self._sync_block_table()

    def _preempt(self, row: int):
        """Take a decoding row out: keep what it generated, give its pages back, queue it for recomputation."""
        r = self.rows[row]
        prompt, sp, _ = self._req[r.request_id]
        n = int(self.gen_count[row].item())
        toks = self.out_tokens[row, :n].tolist()
        lps = self.out_logprobs[row, :n].tolist()
        self.active[row] = 0
        self._release_row(row)
        self.waiting.appendleft(_Pending(r.request_id, prompt, sp, None, r.sample_index, toks, lps))
        self.stats["preemptions"] += 1

    @torch.no_grad()
    def step(self) -> list[RequestOutput]:
        """Admit waiting requests, run prefill work (chunked), run a burst of decode steps for all decoding rows
        (preempting the newest rows when the page pool cannot cover the burst), retire finished rows. Returns the
        requests whose samples have all finished."""
        if self.sleeping:
            self.wake_up()
        finished: list[RequestOutput] = []
        if self.paused:
            return finished
        self._admit()
        self._prefill_work()
        live = [i for i, r in enumerate(self.rows) if r is not None and r.prefilled < 0]
        if not live:
            if self.on_gpu:
                _lib.check_status(self.device)
            return finished
        # ---- decode burst
        left = [self.rows[i].max_tokens - self.rows[i].gen for i in live if self.rows[i].max_tokens > self.rows[i].gen]
        # rows that ignore EOS can only finish at their token limit, which `left` already bounds: nothing can happen
        # inside a longer burst that the host would have to react to, so it is allowed to be several times as long
        # (fewer host round trips between bursts)
        # (only while nothing waits for admission or for its next prefill chunk)
        busy = bool(self.waiting) or any(r is not None and r.prefilled >= 0 for r in self.rows)
        fixed_length = not busy and all(self._req[self.rows[i].request_id][1].ignore_eos for i in live)
        if busy:
            self._quiet_bursts = 0
        # rows that may stop on EOS: the burst grows to 2x and then 4x the check interval while nothing waits and
        # no row has finished for a while (long generations with rare stops), and falls back when one does
        grow = 1 << min(self._quiet_bursts // 2, 2)
        cap = self.check_interval * (8 if fixed_length else (1 if busy else grow))
        steps = max(1, min([cap] + left)) if left else 0
        if steps:
            def short(k):
                return sum(self._pages_short(i, self.rows[i].prompt_len + (self.rows[i].gen - self.rows[i].base) + k)
                           for i in live)

            while steps > 1 and short(steps) > self._free_pages():
                steps = max(1, steps // 2)
            while len(live) > 1 and short(steps) > self._free_pages():
                victim = max(live, key=lambda i: self.rows[i].order)
                self._preempt(victim)
                live.remove(victim)
            if short(steps) > self._free_pages():
                raise RuntimeError("the KV cache cannot hold a single sequence of this length; raise num_pages")
        B = self._bucket(max(live) + 1)
        changed = False
        for i in live:
            r = self.rows[i]
            changed |= self._ensure_pages(i, r.prompt_len + (r.gen - r.base) + steps)
        if changed or self._table_dirty:
            self._sync_block_table()
        for _ in range(steps):
            self._run_decode(B)
        self.decode_steps += steps
        for i in live:
            self.rows[i].gen = min(self.rows[i].gen + steps, self.rows[i].max_tokens)
        # ---- retirement
        act = self.active[:B].cpu()
        done_rows = [i for i in live if act[i] == 0]
        self._quiet_bursts = 0 if done_rows else self._quiet_bursts + 1
        if done_rows:
            gcount = self.gen_count[:B].cpu()
            idx = torch.tensor(done_rows, device=self.device)
            toks = self.out_tokens[idx].cpu()
            lps = self.out_logprobs[idx].cpu()
            for k, i in enumerate(done_rows):
                r = self.rows[i]
                prompt, sp, parts = self._req[r.request_id]
                n = int(gcount[i])
                tl = toks[k, :n].tolist()
                hit_eos = bool(tl) and tl[-1] == self.eos and not sp.ignore_eos
                reason = "stop" if hit_eos else "length"
                lpl = lps[k, :n].tolist()
                lp_out = [{t: Logprob(l)} for t, l in zip(tl, lpl)] if sp.logprobs is not None else None
                parts[r.sample_index] = CompletionOutput(r.sample_index, tl, lp_out, reason,
                                                         cumulative_logprob=float(sum(lpl)), logprob_values=lpl)
                if self.enable_prefix_caching and not self.mrope:
                    # the KV of every token but the last sampled one is in the row's pages: a follow-up request
                    # that re-sends this conversation (multi-turn agents) finds its whole pages in the cache
                    ctx = list(prompt) + tl
                    self._cache_insert(ctx, r.pages, (len(ctx) - 1) // PAGE)
                self._release_row(i)
                if len(parts) == sp.n:
                    finished.append(RequestOutput(r.request_id, list(prompt), [parts[j] for j in range(sp.n)]))
                    del self._req[r.request_id]
        if self.on_gpu:
            _lib.check_status(self.device)
        if _DEBUG:
            self.check_invariants()
        return finished

    def check_invariants(self):
        """Debug check of the scheduler's bookkeeping against the device state (``OPENRLHF_B200_DEBUG=1`` runs it after
        every step): every page of a live row is inside the pool and owned only by rows that share it on purpose, the
        device block table of a decoding row equals the host's, its write slot lies in its own pages, and inactive
        rows write to the dummy page. Raises AssertionError with the offending row."""
        owners: dict[int, list] = {}
        for i, r in enumerate(self.rows):
            if r is None:
                continue
            assert len(set(r.pages)) == len(r.pages), f"row {i} holds a page twice: {r.pages}"
            for idx, pg in enumerate(r.pages):
                assert 0 < pg < self.num_pages, f"row {i} holds page {pg} outside the pool"
                owners.setdefault(pg, []).append((i, idx))
        for pg, own in owners.items():
            if len(own) > 1:
                assert len({idx for _, idx in own}) == 1 and len({self.rows[i].request_id for i, _ in own}) == 1 \
                    or pg in self._cache_hash, f"page {pg} is held by unrelated rows {own}"
        bt = self.block_table.cpu()
        slots, pos, act = self.slots.cpu(), self.pos.cpu(), self.active.cpu()
        hold = {r for _, rows, _ in self._prefilling for r in rows}
        for i, r in enumerate(self.rows):
            decoding = r is not None and i not in hold and r.prefilled < 0
            if decoding and int(act[i]):
                assert bt[i, : len(r.pages)].tolist() == r.pages, f"row {i}: device block table differs from the host's"
                assert int(slots[i]) // PAGE == r.pages[int(pos[i]) // PAGE], f"row {i}: write slot outside its pages"
            elif not decoding and not self._table_dirty and not self._stale_rows:
                assert int(slots[i]) // PAGE == self.dummy_page or r is not None, \
                    f"inactive row {i} writes to page {int(slots[i]) // PAGE}"
        return True

    @torch.no_grad()
    def generate(self, prompt_token_ids: list[list[int]], sampling_params: SamplingParams | list[SamplingParams],
                 request_ids: list | None = None, multi_modal_data: list | None = None) -> list[RequestOutput]:
        """Blocking batch generation on top of the request API (requests wait when rows or KV pages run out).
        multi_modal_data: per prompt None or the dict `add_request` takes."""
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompt_token_ids)
        if sampling_params and sampling_params[0].seed is not None:
            self.seed = sampling_params[0].seed
        base = self._batch_counter
        self._batch_counter += len(prompt_token_ids)
        keys = [("batch", base + i) for i in range(len(prompt_token_ids))]
        mmd = multi_modal_data or [None] * len(keys)
        for k, p, sp, mm in zip(keys, prompt_token_ids, sampling_params, mmd):
            self.add_request(k, p, sp, mm)
        got: dict = {}
        while len(got) < len(keys):
            for ro in self.step():
                got[ro.request_id] = ro
        outs = []
        for i, k in enumerate(keys):
            ro = got[k]
            ro.request_id = request_ids[i] if request_ids else i
            outs.append(ro)
        return outs

    def _start_rows(self, logits: torch.Tensor, entries: list):
        """Contexts whose prefill is complete: copy the open page to the other samples of each request, draw the first
        token of every row from the last-position logits and initialise the rows' device state."""
        dev = self.device
        groups = [rows for _, rows, _ in entries]
        sps = [e.sp for e, _, _ in entries]
        lens = [len(tokens) for _, _, tokens in entries]
        for (e, rows, tokens) in entries:
            n_full = len(tokens) // PAGE
            if self.enable_prefix_caching and e.mm is None:
                self._cache_insert(tokens, self.rows[rows[0]].pages, n_full)
            if len(tokens) % PAGE and len(rows) > 1:
                src = self.rows[rows[0]].pages[n_full]
                for r in rows[1:]:
                    dst = self.rows[r].pages[n_full]
                    self.kv[:, :, dst * PAGE:(dst + 1) * PAGE].copy_(self.kv[:, :, src * PAGE:(src + 1) * PAGE])
            if self.mrope and len(rows) > 1:
                self.rope_delta[rows[1:]] = self.rope_delta[rows[0]]
        rep = torch.tensor([len(g) for g in groups], device=dev)
        rows = torch.tensor([r for g in groups for r in g], dtype=torch.int64, device=dev)
        lg = logits.repeat_interleave(rep, dim=0)                    # one row per sample
        per_row = lambda f, dt: torch.tensor([f(sp, e) for (e, g, _), sp in zip(entries, sps) for _ in g], dtype=dt,
                                             device=dev)
        temps = per_row(lambda sp, e: sp.temperature, torch.float32)
        topk = per_row(lambda sp, e: int(sp.top_k), torch.int32)
        topp = per_row(lambda sp, e: float(sp.top_p), torch.float32)
        tok, lp = sample(lg, temperature=temps, top_k=topk, top_p=topp, seed=self.seed ^ 0x5DEECE66D,
                         step=int(self.decode_steps) * 4096 + int(groups[0][0]))
        plen = torch.tensor([n for n, g in zip(lens, groups) for _ in g], dtype=torch.int32, device=dev)
        base = per_row(lambda sp, e: len(e.done_tokens), torch.int32)
        maxt = torch.tensor([self.rows[r].max_tokens for g in groups for r in g], dtype=torch.int32, device=dev)
        mint = per_row(lambda sp, e: sp.min_tokens, torch.int32)
        ign = per_row(lambda sp, e: sp.ignore_eos, torch.bool)
        for (e, g, _) in entries:                                    # what a preempted sample had generated before
            if e.done_tokens:
                k = len(e.done_tokens)
                self.out_tokens[g[0], :k] = torch.tensor(e.done_tokens, dtype=torch.int64, device=dev)
                self.out_logprobs[g[0], :k] = torch.tensor(e.done_logprobs, dtype=torch.float32, device=dev)
        bl = base.long()
        self.out_tokens[rows, bl] = tok
        self.out_logprobs[rows, bl] = lp
        gc = base + 1
        done = ((tok == self.eos) & ~ign & (mint <= gc)) | (maxt <= gc)
        self.tok[rows] = tok
        self.pos[rows] = plen
        self.seq_lens[rows] = plen + 1
        self.gen_count[rows] = gc
        self.max_tok[rows] = maxt
        self.min_tok[rows] = mint
        self.ignore_eos[rows] = ign
        self.temperature[rows] = temps
        self.top_k_rows[rows] = topk
        self.top_p_rows[rows] = topp
        self.active[rows] = (~done).int()
        page = self.block_table[rows].gather(1, (plen.long() // PAGE)[:, None]).squeeze(1)
        self.slots[rows] = (page * PAGE + (plen % PAGE)).int()
        for g in groups:
            for r in g:
                self.rows[r].gen = self.rows[r].base + 1
                self.rows[r].prefilled = -1


# ---------------------------------------------------------------------------------------------- decode GEMM
_BN64_MAX_N = 2048      # widest output for which 64-column tiles (more CTAs) beat 128-column tiles at short K


def gemm_to_workspace(x: torch.Tensor, w: torch.Tensor, ws: torch.Tensor | None = None):
    """Split-K projection for small M whose fp32 slabs stay in the shared workspace for the next kernel to reduce.
    Returns (workspace, number of slabs). `ws`: use this buffer (a symmetric one under tensor parallelism)."""
    from ..ops.gemm import splitk_workspace

    M, K = x.shape
    N = w.shape[0]
    # narrow N tiles give more CTAs for short K; with a long K (down_proj) 128-wide tiles halve the activation re-reads
    # per weight byte and twice as many K splits keep all SMs streaming (14.4 us vs 16.9 us at N 1536, K 8960)
    bn = 64 if (N <= _BN64_MAX_N and K < 4096) else 128      # small matrices only (e.g. 1536 x 1536): more CTAs
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    kb = (K + 63) // 64
    splits = max(1, min(148 // max(tiles, 1), kb // 4))
    per = (kb + splits - 1) // splits
    splits = (kb + per - 1) // per
    if ws is None:
        ws = splitk_workspace(x.device, splits * M * N)
    assert ws.numel() >= splits * M * N
    gemm(x, w, out=ws, k_splits=splits, split_stride=M * N, bn=bn)
    return ws, splits




def decode_gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
    """Small-M linear for the decode loop: picks a narrow N tile and split-K so that all SMs stream weights."""
    from ..ops.gemm import gemm_splitk

    M, K = x.shape
    N = w.shape[0]
    if not x.is_cuda:
        return F.linear(x, w, bias, residual)
    if M > 256:
        return gemm(x, w, bias=bias, residual=residual)
    bn = 64 if (N <= _BN64_MAX_N and K < 4096) else 128
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    kb = (K + 63) // 64
    splits = max(1, min(148 // max(tiles, 1), kb // 4))
    if splits <= 1:
        return gemm(x, w, bias=bias, residual=residual, bn=bn)
    return gemm_splitk(x, w, splits, bias=bias, residual=residual, bn=bn)
