"""The serving engine: C++ continuous batcher + paged KV pool + model + CUDA-graph decode steps.

Reference parity (behaviour, not structure):
  * ``Executor::{enqueue, step, generate_batch}`` (src/engine/executor_api.rs:540-580, executor_step.rs:113-255)
  * decode first, prefill backfill, phase-isolated launches (src/scheduler/batcher.rs:217-293, SPEC 32)
  * stop on EOS or max_new_tokens (src/engine/executor_step.rs:1464-1471); length guard
    ``prompt + max_new <= max positions`` (src/engine/executor.rs:315-325)
  * per-step hooks Continue / Veto / Terminate (src/engine/executor_step.rs:1406-1455)

B200 design: the host never touches activations. Each decode step is one CUDA-graph replay per batch
bucket; its inputs are a single packed int32 upload from pinned memory (tokens, positions, slot mapping,
context lengths) plus the block tables; its only download is the sampled token per slot. Prefill
chunks run as ordinary launches between decode replays.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from .. import scheduler as S
from ..models.config import ModelConfig
from ..models.decoder import DecoderModel
from ..utils.metrics import GLOBAL as METRICS
from ..utils.tracing import nvtx_range
from .batch import ForwardBatch, GenerateResult, SequenceTelemetry

DECODE_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024)


@dataclass
class EngineConfig:
    max_num_seqs: int = 256
    max_model_len: int = 4096
    max_batch_tokens: int = 8192
    prefill_chunk: int = 8192
    num_pages: int = 0                 # 0 = size from memory_fraction
    memory_fraction: float = 0.85
    enable_prefix_cache: bool = True
    use_cuda_graphs: bool = True
    pages_per_split: int = 32
    seed: int = 0
    order: int = S.ORDER_STRICT_REQUEST_ID
    # swap tier: > 0 turns preemption from "recompute later" into "copy the victim's KV pages to pinned host memory and
    # bring them back when pages are free" (victims chosen by the HGAL policy); overflow goes to the NVMe file
    swap_space_pages: int = 0
    swap_path: Optional[str] = None
    swap_nvme_pages: int = 0
    # a 4-bit tier in front of the host: preempted sequences are first packed into a byte pool on the GPU itself
    # (3.1x smaller than bf16, no PCIe traffic, lossy) and unpacked when they resume; when the pool is full they go
    # to the host as before. Takes effect together with swap_space_pages > 0.
    kv_kivi_pool_pages: int = 0
    # engine.callbacks.CallbackChain run on the residual stream of every forward (RAG / knowledge injection, probes that
    # veto, early exit). Steps then run eagerly (no CUDA graphs). The stock callbacks look at the last row of the step,
    # i.e. they are meant for one request at a time (max_num_seqs = 1); a veto ends every request of the step.
    callbacks: Optional[object] = None
    # debug serving: eager steps with a NaN / Inf check of the residual stream after every layer and of the logits
    # (engine/guard.py::NanTrap; FloatingPointError names the first offender; tensors are dumped to GLLM_DUMP_DIR)
    debug: bool = False
    # every this many engine steps the attention telemetry of the running sequences' KV pages is sampled into the page
    # headers and each request's importance score is refreshed (engine/kv_telemetry.py); 0 = never
    kv_telemetry_every: int = 0
    # prefill chunk size follows the share of free KV pages (64 tokens under a quarter free, ``prefill_chunk`` above three
    # quarters, linear in between) instead of always taking ``prefill_chunk``
    adaptive_prefill_chunk: bool = False
    # speculative decoding by prompt lookup: up to this many draft tokens per sequence and step (0 = off)
    speculative_tokens: int = 0
    speculative_ngram: int = 3
    speculative_max_batch: int = 32    # no speculative steps while more sequences than this are decoding
    # multi-token prediction: use the model's MTP heads (when the checkpoint has them) as the draft source; every step
    # verifies the previous step's candidates (0 = off)
    mtp_depth: int = 0
    # role of this engine in a prefill / decode disaggregated deployment (parallel/pd.py): "collocated",
    # "prefill_only" (finished prefills are handed to `pd_link` with their KV pages) or "decode_only"
    pd_role: str = "collocated"
    # runtime heuristics: decode batch buckets follow the observed batch sizes (runtime/buckets.py), captured graphs
    # live in a budgeted registry (runtime/variants.py), and a background director (runtime/director.py) turns
    # sustained drift of the batch size into a re-derivation of the buckets
    adaptive_buckets: bool = False
    graph_budget_bytes: int = 8 << 30
    director: bool = False


@dataclass
class _ReqState:
    t_submit: float
    t_first: float = 0.0
    t_last: float = 0.0
    hook: Optional[Callable] = None
    stream: Optional[Callable] = None
    n_out: int = 0


class LLMEngine:
    def __init__(self, model: DecoderModel, cfg: EngineConfig = None, tokenizer=None, lockstep_group=None, pd_link=None,
                 pp=None):
        """``lockstep_group``: a process group whose ranks serve DIFFERENT requests but share collective kernels
        inside the model (data-parallel attention + expert-parallel MoE). Every rank then runs the same sequence of
        forwards per step (a rank without work runs an empty one), agreed on by one tiny all-reduce per step."""
        self.model, self.cfg, self.tokenizer = model, cfg or EngineConfig(), tokenizer
        self.lockstep = lockstep_group
        self.pp = pp                           # engine/pp.py PipelineContext: this engine runs one pipeline stage
        self.pd_link = pd_link                 # engine/pd.py link: where a prefill_only engine sends, a decode_only one polls
        self._pd_prompts: Dict[int, List[int]] = {}
        self.mc: ModelConfig = model.cfg
        self.device = model.device
        ec = self.cfg
        ec.max_model_len = min(ec.max_model_len, model.max_positions)
        self.nan_trap = None
        if ec.debug:
            from .callbacks import CallbackChain
            from .guard import NanTrap, nan_check_callback
            self.nan_trap = NanTrap(enabled=True)
            chain = ec.callbacks if ec.callbacks is not None else CallbackChain([])
            chain.add(nan_check_callback(self.nan_trap))
            ec.callbacks = chain
        if ec.callbacks is not None or getattr(model, "expert_pager", None) is not None:
            ec.use_cuda_graphs = False      # host decisions inside the forward (callback chain, expert paging): eager steps
        self.max_blocks = (ec.max_model_len + 15) // 16
        self.num_pages = ec.num_pages or self._auto_pages()
        self.kv_caches = model.alloc_kv_cache(self.num_pages)
        pc = S.PolicyConfig()
        pc.max_batch_size = ec.max_num_seqs
        pc.max_batch_tokens = ec.max_batch_tokens
        pc.prefill_chunk = ec.prefill_chunk
        pc.enable_prefix_cache = ec.enable_prefix_cache
        pc.order = ec.order
        pc.preempt_swap = ec.swap_space_pages > 0
        pc.adaptive_chunk = bool(ec.adaptive_prefill_chunk)
        self.batcher = S.ContinuousBatcher(self.num_pages, 16, ec.max_num_seqs, self.max_blocks, pc)
        self.kv_swap = None
        if ec.swap_space_pages > 0:
            from .kv_swap import KvSwapManager
            self.kv_swap = KvSwapManager(self.kv_caches, ec.swap_space_pages, swap_path=ec.swap_path,
                                         nvme_pages=ec.swap_nvme_pages, device_pool_pages=ec.kv_kivi_pool_pages)
            self.kv_swap.tier_policy = self._swap_tier
        self.kv_telemetry = None
        if ec.kv_telemetry_every > 0:
            from .kv_telemetry import KvTelemetry
            self.kv_telemetry = KvTelemetry(self)
            if self.kv_swap is not None:      # per-page tiers for the packed tier come from the sampled page headers
                hdr = self.kv_telemetry.headers.h
                self.kv_swap.page_tier = lambda page: (int(hdr["precision_tier"][page]) if int(hdr["ref_count"][page]) else 2)
        self._sessions = set()                # requests that belong to a multi-turn session (conversation pipeline)
        self.kv_importance: Dict[int, int] = {}      # request -> importance score 0..255 (callers / telemetry may set it)
        self.ms = ec.max_num_seqs
        dev = self.device
        cuda = dev.type == "cuda"
        pin = dict(pin_memory=True) if cuda else {}
        # host staging (pinned) and device mirrors
        self.h_dec = torch.zeros(4 * self.ms, dtype=torch.int32, **pin)
        self.h_bt = torch.zeros((self.ms, self.max_blocks), dtype=torch.int32, **pin)
        self.h_params = torch.zeros((self.ms, 4), dtype=torch.float32, **pin)
        self.h_out = torch.zeros(self.ms, dtype=torch.int32, **pin)
        self.d_dec = torch.zeros(4 * self.ms, dtype=torch.int32, device=dev)
        self.d_bt = torch.zeros((self.ms, self.max_blocks), dtype=torch.int32, device=dev)
        self.d_params = torch.zeros((self.ms, 4), dtype=torch.float32, device=dev)
        self.d_out = torch.zeros(self.ms, dtype=torch.int32, device=dev)
        self.d_offsets = torch.zeros(self.ms, dtype=torch.int64, device=dev)
        # the kernels' status word (bounded-wait timeouts, bad page / expert ids): copied to pinned memory with every
        # step's tokens and checked before the tokens are committed
        self.d_status = None
        self.h_status = torch.zeros(16, dtype=torch.int32, **pin)
        if cuda:
            from ..ops import _native as nv
            self.d_status = nv.error_word_tensor(dev)
        self.unhealthy: Optional[str] = None
        self.slot_params = np.zeros((self.ms, 4), dtype=np.float32)
        # prefill staging (allocated once: no per-step pinned allocation, concatenation or tensor construction)
        pf_ints = 3 * ec.max_batch_tokens + 5 * self.ms + 64
        self.h_pf = torch.zeros(pf_ints, dtype=torch.int32, **pin)
        self.d_pf = torch.zeros(pf_ints, dtype=torch.int32, device=dev)
        self.h_pf_bt = torch.zeros((self.ms, self.max_blocks), dtype=torch.int32, **pin)
        self.d_pf_bt = torch.zeros((self.ms, self.max_blocks), dtype=torch.int32, device=dev)
        self.h_pf_params = torch.zeros((self.ms, 4), dtype=torch.float32, **pin)
        self.d_pf_params = torch.zeros((self.ms, 4), dtype=torch.float32, device=dev)
        self.h_pf_out = torch.zeros(self.ms, dtype=torch.int32, **pin)
        self.d_pf_out = torch.zeros(self.ms, dtype=torch.int32, device=dev)
        # Split the KV range of a sequence across CTAs only when (sequences x kv heads) alone cannot fill
        # the machine: an unsplit flash-decode CTA streams its pages at full speed, splits add a merge
        # (measured at 256 sequences x 1 kv head, ragged contexts: unsplit 39.9 us, 3 splits 42.1 us).
        want_splits = max(1, -(-3 * 148 // 2 // max(1, self.ms * model.n_kv_local)))
        pps = ec.pages_per_split if want_splits > 1 else 1 << 20
        if want_splits > 1:
            pps = max(8, -(-self.max_blocks // want_splits))
        max_splits = max(1, -(-self.max_blocks // pps))
        self.decode_ws = (ops.DecodeWorkspace(self.ms, model.n_q_local, model.n_kv_local, max_splits, dev)
                          if cuda and self.mc.head_dim == 128 else None)
        if self.decode_ws is not None:
            self.decode_ws.pages_per_split = pps
        model.workspace(max(ec.max_batch_tokens, self.ms))
        if pp is not None:
            self.pp_hidden = torch.zeros((max(ec.max_batch_tokens, self.ms), self.mc.hidden_size), dtype=model.dtype, device=dev)
            ec.use_cuda_graphs = False      # the stage-to-stage transfers run as ordinary p2p calls between the launches
        self.graphs: Dict[int, "torch.cuda.CUDAGraph"] = {}
        from ..runtime.buckets import GoldenBuckets
        from ..runtime.director import Director, DirectorSharedState
        from ..runtime.variants import VariantRegistry
        sizes = sorted({min(b, self.ms) for b in DECODE_BUCKETS})
        self.buckets = GoldenBuckets(buckets=sizes, max_buckets=max(12, len(sizes)))
        self.variants = VariantRegistry(ec.graph_budget_bytes)
        self.director_state = DirectorSharedState()
        self.director = None
        self._evolve_pending = False
        if ec.director:
            self.director = Director(self.director_state, on_event=self._on_director_event, interval_s=1.0).spawn()
        self.reqs: Dict[int, _ReqState] = {}
        self.results: Dict[int, GenerateResult] = {}
        self._next_id = 0
        self.stats = dict(decode_steps=0, prefill_steps=0, decode_tokens=0, prefill_tokens=0, h2d_bytes=0,
                          d2h_bytes=0, kernel_launches=0, preemptions=0)
        self.launches_per_graph: Dict[int, int] = {}
        self.gen = torch.Generator().manual_seed(ec.seed)
        self._all_greedy = True
        self._topk_cap = 0      # tensor parallel, every sampling row has 0 < top_k <= 64: candidates instead of the vocabulary
        self._req_params: Dict[int, tuple] = {}
        from ..scheduler.request_state import RequestStateTable
        self.req_table = RequestStateTable(self.ms, self.device)
        self._slot_of: Dict[int, int] = {}
        # per-slot token counters and timestamps of the decode fast path: one vector update per step; requests with a
        # hook, a stream callback or a draft index are the only ones that still get per-token Python work
        self._sl_nout = np.zeros(self.ms, np.int64)
        self._sl_tfirst = np.zeros(self.ms, np.float64)
        self._sl_tlast = np.zeros(self.ms, np.float64)
        self._sl_slow = np.zeros(self.ms, bool)
        self._req_limits: Dict[int, tuple] = {}
        self._vetoed: Dict[int, str] = {}
        self._spec_idx: Dict[int, object] = {}      # request -> n-gram index of its prompt + generated tokens
        self.spec_stats = dict(steps=0, drafted=0, accepted=0, emitted=0)
        self.mtp = None                             # MtpExecutor: candidates of the model's own heads as drafts
        self._mtp_cand: Dict[int, List[int]] = {}
        if ec.mtp_depth > 0 and getattr(model, "mtp_heads", None):
            from ..speculative.mtp_executor import MtpExecutor
            self.mtp = MtpExecutor(min(ec.mtp_depth, len(model.mtp_heads)))
        # when speculation pays: off for large batches (compute bound), under memory pressure, or once the acceptance
        # average has fallen too low; the draft length follows the acceptance average (speculative/engine.py)
        from ..speculative.engine import SpecDecodingState, SpecMode
        self.spec_state = SpecDecodingState(mode=SpecMode.NGRAM, max_batch_for_spec=max(32, ec.speculative_max_batch))
        self.eagle = None                           # speculative.heads.EagleHead (attach_eagle): feature-level drafts
        self.eagle_depth = 0
        self._eagle_feat: Dict[int, torch.Tensor] = {}      # request -> hidden state behind its last committed token

    # ------------------------------------------------------------------------------------------
    def generate_with_mtp(self, prompt_ids: List[int], max_tokens: int = 256, temperature: float = 0.0, top_k: int = 0,
                          top_p: float = 1.0, eos_ids=None) -> dict:
        """One request through the multi-token-prediction path: the model's MTP heads propose candidates behind every
        committed token, the next step's forward verifies them, rejected ones are rolled back. Returns
        ``{"committed_tokens", "total_mtp_candidates", "total_mtp_accepted", "steps", "finish_reason"}``. Without MTP
        heads (or with ``mtp_depth`` 0) it is an ordinary generation with zero candidates; sampling requests
        (temperature > 0) do not speculate. Reference: generate_with_mtp / MtpGenerateResult
        (src/engine/executor_api.rs:178-260, src/engine/mtp_executor.rs:15-40)."""
        before = dict(self.spec_stats)
        rid = self.add_request(prompt_ids, max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                               eos_ids=eos_ids)
        while rid not in self.results and self.has_work():
            self.step()
        res = self.results.pop(rid)
        st = self.spec_stats
        return {"committed_tokens": list(res.token_ids), "total_mtp_candidates": st["drafted"] - before["drafted"],
                "total_mtp_accepted": st["accepted"] - before["accepted"], "steps": st["steps"] - before["steps"],
                "finish_reason": res.finish_reason}

    def rebalance_experts(self, reduce: bool = True) -> List[int]:
        """Expert load balancing for the expert-sharded tensor-parallel MoE mode: the load balancer's window (summed
        over the ranks with ``reduce``) names the hot experts, which are then mirrored on every rank so that their rows
        are shared out (``MoeLayerWeights.set_mirrors``); captured decode graphs are dropped because the expert stacks
        and block tables change. A collective over the tensor-parallel group: every rank calls it at the same point of
        its (identical) schedule. Returns the hot experts now mirrored."""
        st = self.coordinators.observability.capture_expert_load(reduce=reduce)
        hot = sorted(st["hot_experts"]) if st else []
        layers = [lw.moe for lw in self.model.layers if getattr(lw, "moe", None) is not None
                  and lw.moe.tp_experts is not None and lw.moe.bs_fmt is None]
        if not layers or tuple(hot) == tuple(layers[0].mirrored):
            return list(layers[0].mirrored) if layers else []
        for m in layers:
            m.set_mirrors(hot, self.model)
        self.graphs.clear()
        self.stats["expert_rebalances"] = self.stats.get("expert_rebalances", 0) + 1
        return hot

    def attach_eagle(self, head, depth: int = 3):
        """Draft with an EAGLE head: it continues the target's last hidden feature and the last token for ``depth``
        steps; the target verifies the chain in one forward, so the output stays the target's greedy output. Verify
        steps run eagerly (the feature behind the last kept token is read back from them).
        Reference: EAGLE feature-head drafts (src/speculative/engine.rs:29-420)."""
        self.eagle, self.eagle_depth = head, int(depth)

    def _auto_pages(self) -> int:
        per_page = 16 * self.mc.kv_bytes_per_token(self.model.tp_size) * len(self.model.layer_ids) // max(
            self.mc.num_layers, 1)
        if self.device.type != "cuda":
            return max(64, min(4096, (self.cfg.max_num_seqs * self.cfg.max_model_len) // 16 + 8))
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(free - (1.0 - self.cfg.memory_fraction) * total)
        want = self.cfg.max_num_seqs * self.max_blocks + 64
        return int(max(64, min(want, budget // max(per_page, 1))))

    # ------------------------------------------------------------------------------------------
    def add_request(self, prompt_ids: List[int], *, max_tokens=256, temperature=0.7, top_k=0, top_p=1.0,
                    eos_ids=None, session_id: Optional[str] = None, hook=None, stream=None,
                    request_id: Optional[int] = None) -> int:
        if len(prompt_ids) == 0:
            raise ValueError("empty prompt")
        if len(prompt_ids) + max_tokens > self.cfg.max_model_len:
            raise ValueError(f"SequenceTooLong: {len(prompt_ids)} + {max_tokens} > {self.cfg.max_model_len}")
        rid = self._next_id if request_id is None else request_id
        self._next_id = max(self._next_id, rid) + 1
        eos = list(self.mc.eos_token_ids) if eos_ids is None else list(eos_ids)
        sp = S.SamplingParams(temperature=float(temperature), top_k=int(top_k), top_p=float(top_p),
                              max_new_tokens=int(max_tokens), eos_ids=eos)
        self.batcher.add_request(rid, [int(t) for t in prompt_ids], sp, session_id or "")
        self.reqs[rid] = _ReqState(t_submit=time.perf_counter(), hook=hook, stream=stream)
        if session_id:
            self._sessions.add(rid)
        if self.cfg.pd_role == "prefill_only":
            self._pd_prompts[rid] = [int(t) for t in prompt_ids]
            self._req_params[rid] = (float(temperature), int(top_k), float(top_p))
            self._pd_meta = getattr(self, "_pd_meta", {})
            self._pd_meta[rid] = dict(max_tokens=int(max_tokens), temperature=float(temperature), top_k=int(top_k),
                                      top_p=float(top_p), eos_ids=eos)
        if self.cfg.speculative_tokens > 0:
            from ..speculative.tree import NgramIndex
            idx = NgramIndex(min_n=2, max_n=max(2, self.cfg.speculative_ngram))
            idx.extend(prompt_ids)
            self._spec_idx[rid] = idx
        self._req_params[rid] = (float(temperature), int(top_k), float(top_p))
        self._req_limits[rid] = (int(max_tokens), int(eos[0]) if eos else -1)
        return rid

    submit = add_request

    def _swap_tier(self, rid: int):
        """Precision tier in which a preempted request's KV pages may wait: the KV optimiser's decision from the
        request's importance score and pipeline (a session's pages never drop below fp8, so they go to the host
        unchanged; scratch requests may wait as 4-bit pages on the device)."""
        from ..scheduler.kv_optimizer import decide_tier
        from ..scheduler.types import KvPipeline
        pipeline = KvPipeline.CONVERSATION if rid in self._sessions else KvPipeline.WORKING
        return decide_tier(int(self.kv_importance.get(rid, 100)), pipeline)

    def abort(self, rid: int, reason: str = "aborted") -> bool:
        """Cancel a waiting or running request: it ends at the next step with ``finish_reason = reason`` and the tokens
        it has so far; its pages (and swap copies) are released. False when the request is unknown or already done."""
        if rid not in self.reqs:
            return False
        self._vetoed[rid] = reason
        return True

    def has_work(self) -> bool:
        return bool(self.reqs)

    # ------------------------------------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        return min(self.buckets.bucket_for(n), self.ms)

    def _on_director_event(self, ev):
        """Director thread: the batch size has drifted for several windows in a row -> re-derive the buckets at the next
        step (on the serving thread: graph capture is not thread-safe)."""
        if ev.kind == "bucket_drift":
            self._evolve_pending = True

    def evolve_buckets(self):
        """Re-derive the decode buckets from the observed batch sizes; graphs of new buckets are captured on first use,
        graphs of dropped buckets leave the registry when its budget needs the room."""
        before = list(self.buckets.buckets)
        after = self.buckets.evolve()
        self._evolve_pending = False
        return before, list(after)

    def _decode_batch(self, B: int) -> ForwardBatch:
        ms = self.ms
        return ForwardBatch(token_ids=self.d_dec[0:B], positions=self.d_dec[ms:ms + B],
                            slot_mapping=self.d_dec[2 * ms:2 * ms + B], block_tables=self.d_bt[:B],
                            ctx_lens=self.d_dec[3 * ms:3 * ms + B], is_decode=True)

    def _pp_forward(self, batch, T: int, **kw):
        """One pipeline stage of a forward over ``T`` tokens: hidden states in from the previous stage, out to the
        next; only the last stage returns logits (the others return None)."""
        pp = self.pp
        hidden_in = None
        if not pp.is_first:
            hidden_in = pp.recv_hidden(self.pp_hidden[:T])
        out = self.model.forward(batch, self.kv_caches, hidden_in=hidden_in, **kw)
        if not pp.is_last:
            pp.send_hidden(out[:T])
            return None
        return out

    def _ep_bound(self, decode: bool):
        """Expert parallelism: how many tokens ANY rank may route in this kind of step (the same number on every rank:
        it sizes the grouped-GEMM grids over the rows a rank receives). Decode steps are bounded by the slot count,
        prefill steps by the token budget; without this the GEMMs would scan the row blocks of the largest prefill."""
        ep = getattr(self.model, "ep", None)
        if ep is not None:
            ep.token_bound = min(ep.max_tokens, self.ms if decode else max(self.cfg.max_batch_tokens, self.ms))

    def _decode_body(self, B: int):
        self._ep_bound(True)
        if self.pp is not None:
            logits = self._pp_forward(self._decode_batch(B), B, decode_ws=self.decode_ws)
            if logits is not None:
                self._sample(logits, self.d_params[:B], self.d_offsets[:B], self.d_out[:B])
            self.pp.share_tokens(self.d_out[:B])
            self.d_offsets[:B] += 1
            return
        logits = self.model.forward(self._decode_batch(B), self.kv_caches, decode_ws=self.decode_ws,
                                    **({"callbacks": self.cfg.callbacks} if self.cfg.callbacks is not None else {}))
        self._sample(logits, self.d_params[:B], self.d_offsets[:B], self.d_out[:B])
        self.d_offsets[:B] += 1
        tm = getattr(self.model, "op_timer", None)
        if tm is not None:
            tm.mark("sample")

    def decode_breakdown(self, B: int, replays: int = 3):
        """Per-op device milliseconds of one captured decode step of bucket ``B`` (event nodes inside a fresh graph of
        the same step; the graph used for serving is left as it was)."""
        from ..utils.tracing import GraphTimer
        key = self._graph_key(B)
        keep = self.graphs.get(key)
        self.model.op_timer = GraphTimer()
        trace_k = int(os.environ.get("GLLM_TRACE_K", "0"))   # also stamp the phases of the GEMMs with this K (and N)
        trace_n = int(os.environ.get("GLLM_TRACE_N", "0"))
        trace = None
        if trace_k:
            import ctypes
            from ..ops import _native as nv
            lib = nv.lib()
            if not lib.gllm_gemm_trace_enabled():
                raise RuntimeError("phase stamps need the trace build of the kernel library: python -m gllm_b200.build "
                                   "--trace, then GLLM_TRACE_LIB=1")
            lib.gllm_gemm_set_trace.argtypes = [ctypes.c_void_p]
            lib.gllm_gemm_set_trace.restype = None
            lib.gllm_gemm_set_trace_k.argtypes = [ctypes.c_int]
            lib.gllm_gemm_set_trace_k.restype = None
            trace = torch.zeros(12, dtype=torch.int64, device=self.device)
            lib.gllm_gemm_set_trace_n.argtypes = [ctypes.c_int]
            lib.gllm_gemm_set_trace_n.restype = None
            lib.gllm_gemm_set_trace_k(trace_k)
            lib.gllm_gemm_set_trace_n(trace_n)
            lib.gllm_gemm_set_trace(trace.data_ptr())
        try:
            g = self._capture(B)
            for _ in range(replays):
                g.replay()
            res = self.model.op_timer.results()
            if trace is not None:
                st = trace.tolist()
                res.update({f"_clk{j}": float(st[j + 1] - st[j]) if st[j + 1] and st[j] else 0.0 for j in range(8)})
                if st[9]:       # push all-reduce: flags released -> rows reduced -> all ranks done
                    res.update({"_clk_push_reduce": float(st[9] - st[7]), "_clk_push_finish": float(st[8] - st[9])})
        finally:
            if trace is not None:
                lib.gllm_gemm_set_trace(None)
                lib.gllm_gemm_set_trace_k(0)
                lib.gllm_gemm_set_trace_n(0)
            self.model.op_timer = None
            if keep is not None:
                self.graphs[key] = keep
        self.d_offsets[:B] -= replays
        return res

    def _set_sampling_mode(self, rows):
        """``rows``: [n, 4] host rows {temperature, top_k, top_p, _} of the step's sampling slots."""
        self._all_greedy = bool((rows[:, 0] <= 0).all())
        self._topk_cap = 0
        tp = self.model.tp
        if not self._all_greedy and tp is not None and tp.size > 1:
            k = rows[rows[:, 0] > 0, 1]
            if k.size and bool(((k > 0) & (k <= 64)).all()):
                self._topk_cap = 64

    def _graph_key(self, B):
        return (B, True if self._all_greedy else ("topk" if self._topk_cap else False))

    def _note_callback_veto(self, rids):
        """A callback of the chain vetoed during the last forward: the step's requests end with that reason."""
        from .callbacks import CallbackAction
        if getattr(self.model, "callback_action", None) == CallbackAction.VETO:
            for rid in rids:
                self._vetoed[rid] = "vetoed by a layer callback"

    def _sample(self, logits, params, offsets, out):
        if self.nan_trap is not None:
            self.nan_trap.check("logits", logits)
        tp = self.model.tp
        if tp is not None and tp.size > 1:
            # the greedy fast path (pairs instead of full logit rows) is fixed per captured graph
            tp.sample_vocab_parallel(logits, self.model.vocab_local, self.model.vocab_start, params, self.cfg.seed,
                                     offsets, out, self.mc.vocab_size, greedy=self._all_greedy,
                                     topk_cap=0 if self._all_greedy else self._topk_cap)
        else:
            ops.sample(logits, params, vocab=self.mc.vocab_size, seed=self.cfg.seed, step_offsets=offsets, out=out,
                       generator=self.gen)

    def _run_decode(self, plan) -> np.ndarray:
        ms = self.ms
        plan.pack_decode_into(self.h_dec.numpy())
        self.batcher.copy_slot_block_tables_into(self.h_bt.numpy().reshape(-1))
        ids = plan.dec_seq_ids
        active = np.nonzero(ids >= 0)[0]
        n_slots = int(active[-1]) + 1
        self.buckets.observe(n_slots)
        with self.director_state.lock:
            self.director_state.batch_sizes.add(float(n_slots))
        if self.cfg.adaptive_buckets and (self._evolve_pending or (self.stats["decode_steps"] + 1) % 512 == 0):
            self.evolve_buckets()
        B = self._bucket(n_slots)
        self.h_params.numpy()[:] = self.slot_params
        cuda = self.device.type == "cuda"
        self.d_dec.copy_(self.h_dec, non_blocking=cuda)
        self.d_bt.copy_(self.h_bt, non_blocking=cuda)
        self.d_params.copy_(self.h_params, non_blocking=cuda)
        self.stats["h2d_bytes"] += self.h_dec.numel() * 4 + self.h_bt.numel() * 4 + self.h_params.numel() * 4
        self._set_sampling_mode(self.slot_params)
        if cuda and self.cfg.use_cuda_graphs and self.cfg.callbacks is None:
            key = self._graph_key(B)
            g = self.graphs.get(key)
            if g is None and self.lockstep is None:
                g = self._capture(B)
            if g is not None:
                self._note_variant_hit(key)
                g.replay()
            else:     # lockstep: a capture (with its warm-up run) cannot happen on one rank alone; see precapture()
                self._decode_body(B)
        else:
            self._decode_body(B)
            if self.cfg.callbacks is not None:
                self._note_callback_veto(int(i) for i in plan.dec_seq_ids if i >= 0)
        if self.d_status is not None:
            self.h_status.copy_(self.d_status, non_blocking=True)      # lands before the blocking copy below returns
        self.h_out.copy_(self.d_out, non_blocking=False)
        self.stats["d2h_bytes"] += self.h_out.numel() * 4 + (64 if self.d_status is not None else 0)
        self.stats["decode_steps"] += 1
        self.stats["decode_tokens"] += int(plan.num_decode)
        return self.h_out.numpy()

    # ---- speculative decoding (prompt lookup) ---------------------------------------------------------
    def _run_speculative_decode(self, plan):
        """One verify forward over [last token, draft...] of every running sequence instead of a one-token decode step.
        Drafts come from each request's own history (the continuation that followed the same n-gram earlier: prompt
        lookup); the target's greedy choices decide how many are kept, so the output equals plain greedy decoding.
        Returns (first new token per slot, {request: the further tokens}) or None when nobody had a draft.

        Reference parity: ``draft_phase`` / ``verify_phase`` (src/speculative/engine.rs:310-420), PLD spine and n-gram
        index (src/speculative/tree.rs:93-340,394-452), KV rollback by position (src/engine/mtp_executor.rs)."""
        from ..speculative.verify import verify_greedy
        ids = plan.dec_seq_ids
        pressure = 1.0 - self.batcher.num_free_pages / max(self.batcher.num_total_pages, 1)
        lookup_on = self.spec_state.should_speculate(int((ids >= 0).sum()), pressure)
        k = min(self.cfg.speculative_tokens, self.spec_state.controller.draft_len()) if lookup_on else 0
        slots = [int(sl) for sl in np.nonzero(ids >= 0)[0]]
        drafts, from_mtp = {}, {}
        for sl in slots:
            rid = int(ids[sl])
            d = []
            if self.mtp is not None:        # the model's own candidates from the step before (depth set by the controller)
                d = self._mtp_cand.pop(rid, [])[:self.mtp.active_depth()]
                from_mtp[sl] = bool(d)
            if not d and k > 0:
                idx = self._spec_idx.get(rid)
                cand = idx.lookup(k) if idx is not None else []
                d = [int(t) for t in cand[0][:k]] if cand else []
            if not d and self.eagle is not None and rid in self._eagle_feat:
                tok = torch.tensor([int(plan.dec_tokens[sl])], device=self.device)
                d = [int(t[0]) for t in self.eagle.draft(self._eagle_feat[rid][None], tok, self.eagle_depth)]
                bad = next((i for i, t in enumerate(d) if not 0 <= t < self.mc.vocab_size), len(d))
                d = d[:bad]               # a head reading through a padded lm_head may name a padding row
            left = self._remaining_tokens(rid)
            d = d[:max(0, left - 1)]            # never draft past the request's length limit
            if d and not self.batcher.reserve_tokens(rid, 1 + len(d)):
                d = []
            drafts[sl] = d
        if not any(drafts.values()) and (self.mtp is None or self.mtp.active_depth() == 0) and self.eagle is None:
            return None      # nothing to verify (and no candidates wanted): the captured one-token decode step runs
        self.batcher.copy_slot_block_tables_into(self.h_bt.numpy().reshape(-1))
        bt = self.h_bt.numpy()
        toks, pos, slotmap, q_start, q_len, ctx = [], [], [], [], [], []
        for sl in slots:
            d = drafts[sl]
            p0 = int(plan.dec_positions[sl])
            q_start.append(len(toks))
            q_len.append(1 + len(d))
            ctx.append(p0 + 1 + len(d))
            for i, t in enumerate([int(plan.dec_tokens[sl])] + d):
                toks.append(t)
                pos.append(p0 + i)
                slotmap.append(int(bt[sl, (p0 + i) // 16]) * 16 + (p0 + i) % 16)
        dev = self.device
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        T = len(toks)
        batch = ForwardBatch(token_ids=i32(toks), positions=i32(pos), slot_mapping=i32(slotmap),
                             block_tables=torch.from_numpy(bt[slots]).to(dev), ctx_lens=i32(ctx), is_decode=False,
                             q_start=i32(q_start), q_len=i32(q_len), max_q_len=max(q_len), want_mtp=self.mtp is not None)
        self.stats["h2d_bytes"] += 4 * (3 * T + 3 * len(slots)) + bt[slots].nbytes
        self._ep_bound(False)
        hid = None
        if self.eagle is not None and self.mtp is None:
            hid = self.model.forward(batch, self.kv_caches, return_hidden=True)
            logits = self.model.head_logits(hid)
        else:
            logits = self.model.forward(batch, self.kv_caches)
        out = torch.empty(T, dtype=torch.int32, device=dev)
        greedy = torch.zeros((T, 4), dtype=torch.float32, device=dev)
        zeros = torch.zeros(T, dtype=torch.int64, device=dev)
        keep = self._all_greedy
        self._all_greedy = True
        self._sample(logits, greedy, zeros, out)
        mtp_choice = []
        if self.mtp is not None:      # every row's candidates; the row of the last accepted token is picked below
            for lg in self.model.last_mtp_logits[:self.mtp.depth]:
                o = torch.empty(T, dtype=torch.int32, device=dev)
                self._sample(lg, greedy, zeros, o)
                mtp_choice.append(o.cpu().numpy())
        self._all_greedy = keep
        if self.d_status is not None:
            self.h_status.copy_(self.d_status, non_blocking=True)
        choice = out.cpu().numpy()
        self.stats["d2h_bytes"] += T * 4
        self.stats["decode_steps"] += 1
        first = np.zeros(self.ms, np.int32)
        extra = {}
        st = self.spec_stats
        st["steps"] += 1
        for j, sl in enumerate(slots):
            d = drafts[sl]
            seg = choice[q_start[j]:q_start[j] + q_len[j]]
            n_acc, nxt = verify_greedy(d, seg)
            new = d[:n_acc] + [nxt]
            first[sl] = new[0]
            if len(new) > 1:
                extra[int(ids[sl])] = new[1:]
            st["drafted"] += len(d)
            st["accepted"] += n_acc
            st["emitted"] += len(new)
            if d and not from_mtp.get(sl):
                self.spec_state.record(len(d), n_acc)
            if hid is not None:           # the feature behind the last token that stays: the next draft starts there
                self._eagle_feat[int(ids[sl])] = hid[q_start[j] + n_acc].clone()
            self.stats["decode_tokens"] += len(new)
            if self.mtp is not None:
                if from_mtp.get(sl):
                    self.mtp.controller.update(n_acc, len(d))
                row = q_start[j] + n_acc         # the hidden state behind the last token that stays
                self._mtp_cand[int(ids[sl])] = [int(c[row]) for c in mtp_choice]
        return first, extra

    # ---- prefill / decode disaggregation (engine/pd.py) ------------------------------------------------
    def _export_handoff(self, rid: int, first_token: int):
        """Prefill-only role: ship the request with the KV of its prompt's full pages."""
        from .pd import PdHandoff
        prompt = self._pd_prompts.pop(rid)
        n_full = len(prompt) // 16
        pages = None
        if n_full:
            idx = torch.as_tensor(self.batcher.block_table_of(rid)[:n_full], dtype=torch.long, device=self.device)
            pages = torch.stack([(c.view(torch.uint8) if c.dtype == torch.float8_e4m3fn else c).index_select(0, idx)
                                 for c in self.kv_caches]).contiguous()
        meta = getattr(self, "_pd_meta", {}).pop(rid, dict(max_tokens=256, temperature=0.0, top_k=0, top_p=1.0, eos_ids=[]))
        self.stats["pd_exported"] = self.stats.get("pd_exported", 0) + 1
        if self.pd_link is not None:
            self.pd_link.send(PdHandoff(rid, prompt, first_token, meta, pages))

    def export_prefix_pages(self, tokens: List[int]):
        """(number of cached full pages, their KV [layers, pages, ...]) of the longest cached prefix of ``tokens`` in this
        pool, or (0, None): what a peer needs to continue the same conversation (KV distribution modes)."""
        n_full = len(tokens) // 16
        have = list(self.batcher.lookup_prefix_pages([int(t) for t in tokens[:n_full * 16]])) if n_full else []
        if not have:
            return 0, None
        idx = torch.as_tensor(have, dtype=torch.long, device=self.device)
        pages = torch.stack([(c.view(torch.uint8) if c.dtype == torch.float8_e4m3fn else c).index_select(0, idx)
                             for c in self.kv_caches]).contiguous()
        return len(have), pages

    def import_prefix_pages(self, tokens: List[int], pages) -> int:
        """The first ``pages.shape[1]`` full pages of ``tokens`` become cached prefix pages of this pool (pages already
        cached here are kept as they are). Returns how many pages were written."""
        n = 0 if pages is None else int(pages.shape[1])
        if n == 0:
            return 0
        dst = self.batcher.import_prefix([int(t) for t in tokens[:n * 16]], "")
        sel = [i for i, p in enumerate(dst) if p >= 0]          # -1: that page is already cached here
        if sel:
            src_idx = torch.as_tensor(sel, dtype=torch.long, device=self.device)
            dst_idx = torch.as_tensor([dst[i] for i in sel], dtype=torch.long, device=self.device)
            pages = pages.to(self.device)
            for l, c in enumerate(self.kv_caches):
                tgt = c.view(torch.uint8) if c.dtype == torch.float8_e4m3fn else c
                tgt.index_copy_(0, dst_idx, pages[l].index_select(0, src_idx))
        return len(sel)

    def import_handoff(self, h) -> int:
        """Decode-only role: the prompt's full pages become cached prefix pages of this pool, then the request is
        admitted; its admission finds them and computes only the partial last page before decoding."""
        n_full = len(h.prompt) // 16
        if n_full and h.pages is not None:
            self.import_prefix_pages(h.prompt[:n_full * 16], h.pages)
        self.stats["pd_imported"] = self.stats.get("pd_imported", 0) + 1
        p = h.params
        return self.add_request(h.prompt, max_tokens=p["max_tokens"], temperature=p["temperature"], top_k=p["top_k"],
                                top_p=p["top_p"], eos_ids=p["eos_ids"], request_id=h.request_id)

    def add_request_context_parallel(self, prompt_ids: List[int], cp_rank: int, cp_size: int, group=None, **kw) -> int:
        """A long prompt prefilled by ``cp_size`` engines together (every rank of ``group`` makes this call with the same
        prompt): each rank runs the layers on its page-aligned shard of the prompt's full pages, the ranks exchange
        the KV pages layer by layer (``parallel.context_parallel.CpPrefill``), and every rank ends with the whole
        prompt's pages as cached prefix pages of its own pool. The request is then admitted as usual: it finds the
        pages and computes only the partial last page before decoding, on every rank alike (or on the one rank that
        keeps the request, when the others abort theirs). Falls back to a plain ``add_request`` on all ranks when any
        rank cannot take part (prefix already cached there, too few free pages, a prompt shorter than one page per
        rank). Reference: context-parallel prefill (src/engine/coordinator/context_parallel.rs:76-127, 286-390)."""
        prompt = [int(t) for t in prompt_ids]
        n_full = len(prompt) // 16
        from ..parallel.context_parallel import CpConfig, CpPrefill
        zigzag = n_full >= 4 * cp_size          # balanced causal work once every rank gets two chunks of some size
        ok = (cp_size > 1 and self.cfg.enable_prefix_cache
              and CpPrefill.every_rank_has_tokens(n_full * 16, cp_size, zigzag)
              and not self.mc.is_mla and self.pp is None
              and len(self.batcher.lookup_prefix_pages(prompt[:n_full * 16])) == 0
              and self.batcher.num_free_pages >= n_full + (len(prompt) + int(kw.get("max_tokens", 256))) // 16 + 2)
        if cp_size > 1:
            import torch.distributed as dist
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            ok = bool(int(flag[0]))
        if not ok:
            return self.add_request(prompt, **kw)
        dst = self.batcher.import_prefix(prompt[:n_full * 16], "")
        if len(dst) != n_full or min(dst) < 0:
            raise RuntimeError("context-parallel prefill: the page pool changed between the check and the import")
        bt = torch.tensor([dst], dtype=torch.int32, device=self.device)
        cp = CpPrefill(CpConfig(cp_size, cp_rank), [n_full * 16], bt, group=group, zigzag=zigzag)
        batch = cp.local_batch([prompt[:n_full * 16]])
        self._ep_bound(False)
        self.model.forward(batch, self.kv_caches, return_hidden=True)
        self.stats["cp_prefill_tokens"] = self.stats.get("cp_prefill_tokens", 0) + batch.num_tokens
        self.stats["cp_prefills"] = self.stats.get("cp_prefills", 0) + 1
        return self.add_request(prompt, **kw)

    def _remaining_tokens(self, rid: int) -> int:
        st = self.batcher.state_of(rid)
        if st is None:
            return 0
        return int(st.get("max_new_tokens", 1 << 30)) - int(st.get("num_generated", 0))

    def _capture(self, B: int):
        # One capture stream for all decode graphs, with its own split-K scratch and grid-barrier words: the GEMMs inside
        # the graphs then share nothing with eager launches on other streams (prefill chunks), so the two may overlap.
        # Warm up outside capture so lazy initialisation (attribute setting, descriptor cache) is done.
        if getattr(self, "_graph_stream", None) is None:
            from ..ops import _native as nv_
            self._graph_stream = torch.cuda.Stream(device=self.device)
            nv_.stream_splitk_workspace(self._graph_stream)
        s = self._graph_stream
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._decode_body(B)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.d_offsets[:B] -= 1
        g = torch.cuda.CUDAGraph()
        from ..ops import _native as nv
        n0 = nv.CALLS[0]
        with torch.cuda.graph(g, stream=s):
            self._decode_body(B)
        self.launches_per_graph[B] = nv.CALLS[0] - n0
        self.graphs[self._graph_key(B)] = g
        self._register_variant(self._graph_key(B), g)
        return g

    def _variant_key(self, key):
        from ..runtime.variants import MechanismId, VariantKey
        mech = (MechanismId.DENSE,) if key[1] is True else (MechanismId.DENSE, MechanismId.SAMPLED)
        if key[1] == "topk":          # sampled from per-rank candidates: a graph of its own beside the full-vocabulary one
            mech = mech + (MechanismId.SAMPLED,)
        if self.mc.is_moe:
            mech = mech + (MechanismId.MOE_EP,) if getattr(self.model, "ep", None) is not None else mech
        return VariantKey(int(key[0]), mech)

    def _register_variant(self, key, graph):
        """Captured graphs are budgeted: a graph pins its private memory pool, so cold ones leave when a new one
        would exceed the budget (the reference budgets JIT code in the instruction cache the same way)."""
        from ..runtime.variants import CompiledVariant
        est = int(key[0]) * self.mc.hidden_size * 64 + (8 << 20)      # activations a graph's pool keeps alive
        vk = self._variant_key(key)
        self.variants.register(CompiledVariant(vk, graph, bytes=est))
        live = {v.key for v in self.variants.variants.values()}
        for k in [k for k in self.graphs if self._variant_key(k) not in live]:
            del self.graphs[k]                                         # evicted by the registry: drop the graph

    def _note_variant_hit(self, key):
        v = self.variants.variants.get(self._variant_key(key))
        if v is not None:
            v.hits += 1

    def _run_prefill(self, plan) -> np.ndarray:
        t_host0 = time.perf_counter()
        ev = None
        if self.device.type == "cuda":
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        try:
            return self._run_prefill_inner(plan)
        finally:
            if ev is not None:
                ev[1].record()
                ev[1].synchronize()
                self.stats["prefill_device_ms"] = self.stats.get("prefill_device_ms", 0.0) + ev[0].elapsed_time(ev[1])
            self.stats["prefill_wall_ms"] = self.stats.get("prefill_wall_ms", 0.0) + (time.perf_counter() - t_host0) * 1e3

    def _run_prefill_inner(self, plan) -> np.ndarray:
        dev = self.device
        cuda = dev.type == "cuda"
        T, S_, n_last, max_q = plan.pack_prefill_into(self.h_pf.numpy(), self.h_pf_bt.numpy().reshape(-1))
        used = 3 * T + 3 * S_ + 2 * n_last
        self.d_pf[:used].copy_(self.h_pf[:used], non_blocking=cuda)
        self.d_pf_bt[:S_].copy_(self.h_pf_bt[:S_], non_blocking=cuda)
        self.stats["h2d_bytes"] += used * 4 + S_ * self.max_blocks * 4
        dp = self.d_pf
        o = 3 * T + 3 * S_
        rows = dp[o:o + n_last] if n_last else None
        batch = ForwardBatch(token_ids=dp[0:T], positions=dp[T:2 * T], slot_mapping=dp[2 * T:3 * T],
                             block_tables=self.d_pf_bt[:S_], ctx_lens=dp[3 * T + 2 * S_:3 * T + 3 * S_], is_decode=False,
                             q_start=dp[3 * T:3 * T + S_], q_len=dp[3 * T + S_:3 * T + 2 * S_],
                             max_q_len=int(max_q), logits_rows=rows, want_mtp=self.mtp is not None)
        self.stats["prefill_steps"] += 1
        self.stats["prefill_tokens"] += int(T)
        self.model.op_timer = getattr(self, "prefill_timer", None)   # utils.tracing.GraphTimer(eager=True) or None
        self._ep_bound(False)
        try:
            if self.pp is not None:
                logits = self._pp_forward(batch, T, return_hidden=rows is None)
                if rows is None:
                    return np.zeros(0, np.int32)
            elif rows is None:
                self.model.forward(batch, self.kv_caches, return_hidden=True)
                return np.zeros(0, np.int32)
            else:
                logits = self.model.forward(batch, self.kv_caches,
                                            **({"callbacks": self.cfg.callbacks} if self.cfg.callbacks is not None else {}))
                self._note_callback_veto(int(it.seq_id) for it in plan.prefill)
        finally:
            self.model.op_timer = None
        last_slots = self.h_pf.numpy()[o + n_last:o + 2 * n_last]
        self._set_sampling_mode(self.slot_params[last_slots])
        self.h_pf_params.numpy()[:n_last] = self.slot_params[last_slots]
        self.d_pf_params[:n_last].copy_(self.h_pf_params[:n_last], non_blocking=cuda)
        sl = dp[o + n_last:o + 2 * n_last]
        offs = self.d_offsets.index_select(0, sl)
        out = self.d_pf_out[:n_last]
        if logits is not None:
            self._sample(logits, self.d_pf_params[:n_last], offs, out)
        if self.pp is not None:
            self.pp.share_tokens(out)
        self.d_offsets.index_add_(0, sl, torch.ones(n_last, dtype=torch.int64, device=dev))
        if self.mtp is not None and self.model.last_mtp_logits:
            # the heads' candidates behind each finished prompt: the first decode step of the request verifies them
            greedy = torch.zeros((n_last, 4), dtype=torch.float32, device=dev)
            zeros = torch.zeros(n_last, dtype=torch.int64, device=dev)
            keep, self._all_greedy = self._all_greedy, True
            cands = []
            for lg in self.model.last_mtp_logits[:self.mtp.depth]:
                o = torch.empty(n_last, dtype=torch.int32, device=dev)
                self._sample(lg, greedy, zeros, o)
                cands.append(o.cpu().numpy())
            self._all_greedy = keep
            rids = [int(it.seq_id) for it in plan.prefill if it.last]
            for j, rid in enumerate(rids):
                self._mtp_cand[rid] = [int(c[j]) for c in cands]
        if self.d_status is not None:
            self.h_status.copy_(self.d_status, non_blocking=True)
        self.h_pf_out[:n_last].copy_(out, non_blocking=False)     # the only wait of the step: the sampled tokens
        self.stats["d2h_bytes"] += n_last * 4
        return self.h_pf_out.numpy()[:n_last].copy()

    # ------------------------------------------------------------------------------------------
    def _device_status(self) -> int:
        """Status word as of the last step's download (0 = every kernel finished cleanly)."""
        return int(self.h_status[0])

    def _check_device_status(self, plan):
        """A kernel that gave up a bounded wait (a peer rank that stalled) or met a bad page id leaves garbage behind.
        Nothing of such a step is committed: the running requests fail, the engine is marked unhealthy (a tensor-
        parallel rank must be re-synchronised with ``tp.reset()`` on every rank before it serves again) and the
        caller gets an exception instead of tokens."""
        code = self._device_status()
        if code == 0:
            return
        from ..ops import _native as nv
        if self.d_status is not None:
            self.d_status.zero_()
        self.h_status.zero_()
        name = nv.ERROR_NAMES.get(code, "?")
        self.unhealthy = f"device status {code} ({name})"
        failed = list(self.reqs)          # waiting ones too: this rank serves nothing until it is re-synchronised
        for rid in failed:
            self._vetoed[rid] = f"error: rank unhealthy, {name}"
        self._collect()
        METRICS.inc("device_status_errors")
        raise nv.DeviceStatusError(code, f"in engine step; {len(failed)} request(s) failed")

    # ------------------------------------------------------------------------------------------
    @property
    def coordinators(self):
        """The engine's seams under the reference's coordinator names (dispatch, kv, compute, inference, model context,
        observability): engine/coordinators.py. Built on first use."""
        c = getattr(self, "_coordinators", None)
        if c is None:
            from ..parallel.config import PdRole
            from .coordinators import Coordinators
            role = {"prefill_only": PdRole.PREFILL_ONLY, "decode_only": PdRole.DECODE_ONLY}.get(self.cfg.pd_role, PdRole.COLLOCATED)
            c = self._coordinators = Coordinators.of(self, pd_role=role, swap=getattr(self.kv_swap, "swap", None))
        return c

    def step(self) -> List[GenerateResult]:
        """One scheduler iteration: decode replay for the running set, then one prefill chunk batch."""
        if self.cfg.pd_role == "decode_only" and getattr(self.pd_link, "nonblocking", False):
            for h in self.pd_link.poll():      # a link that never blocks: take what the prefill side has finished
                self.import_handoff(h)
        if self.kv_swap is not None and self.batcher.num_free_pages < max(8, self.num_pages // 16):
            # memory is tight: the batcher's next victims follow the eviction policy, not "youngest first"
            running = [rid for rid in self.reqs if rid not in self.kv_swap.keys and rid not in self.kv_swap.packed]
            self.batcher.set_victim_order(self.kv_swap.victim_order(running))
        self._steps = getattr(self, "_steps", 0) + 1
        if self._steps % 16 == 1:
            # the observability coordinator samples the system state (free pages, fragmentation, queue depths) and
            # hands it to the batcher's policy, as the reference's step loop does through its coordinators
            self.coordinators.observability.capture()
        plan = self.batcher.schedule()
        self.stats["preemptions"] += len(plan.preempted)
        if self.kv_swap is not None:
            # before any kernel of this step runs: the victims' pages may already belong to someone else in this plan
            for it in plan.swap_out:
                self.kv_swap.swap_out(it)
            for it in plan.swap_in:
                self.kv_swap.swap_in(it)
            self.stats["swap_outs"] = self.stats.get("swap_outs", 0) + len(plan.swap_out)
            self.stats["swap_ins"] = self.stats.get("swap_ins", 0) + len(plan.swap_in)
            self.kv_swap.touch(int(i) for i in plan.dec_seq_ids if i >= 0)
        if self.lockstep is not None:
            return self._step_lockstep(plan)
        if plan.idle:
            return self._collect()
        for it in plan.prefill:
            if it.start == 0 or self.slot_params[it.slot, 3] != float(it.seq_id):
                sp = self._params_of(it.seq_id)
                self.slot_params[it.slot] = (sp[0], sp[1], sp[2], float(it.seq_id))
                self._bind_slot(int(it.seq_id), int(it.slot))
        dec_tokens = np.zeros(self.ms, np.int32)
        pf_tokens = np.zeros(0, np.int32)
        spec_extra = {}
        if plan.num_decode > 0:
            spec = None
            if (self.cfg.speculative_tokens > 0 or self.mtp is not None or self.eagle is not None) and bool(
                    (self.slot_params[:, 0] <= 0).all()):
                with nvtx_range("speculative_step"):
                    spec = self._run_speculative_decode(plan)
            if spec is not None:
                dec_tokens, spec_extra = spec
            else:
                with nvtx_range("decode_step"):
                    dec_tokens = self._run_decode(plan).copy()
                if self.mtp is not None:
                    self.mtp.controller.update(0, 0)        # a plain step: counts towards switching the heads back on
                if self.kv_telemetry is not None and self._steps % self.cfg.kv_telemetry_every == 0:
                    self.kv_telemetry.sample(plan, max_sequences=32)      # before a prefill chunk reuses the workspace rows
        if plan.num_prefill_seqs > 0:
            with nvtx_range("prefill_chunk"):
                pf_tokens = self._run_prefill(plan)
        self._check_device_status(plan)
        METRICS.set("kv_free_pages", float(self.batcher.num_free_pages))
        METRICS.set("running_requests", float(len(self.reqs)))
        now = time.perf_counter()
        ids = plan.dec_seq_ids
        # hooks / streaming observe the sampled tokens before they are committed
        live = np.nonzero(ids >= 0)[0]
        self._count_decode(live, ids, dec_tokens, now)
        k = 0
        handoff = []
        for it in plan.prefill:
            if it.last:
                self.req_table.advance(int(it.slot), int(pf_tokens[k]))
                self._observe(int(it.seq_id), int(pf_tokens[k]), now)
                if self.cfg.pd_role == "prefill_only":
                    handoff.append((int(it.seq_id), int(pf_tokens[k])))
                k += 1
        for rid, tok in handoff:               # before the commit: the sequence still owns its pages
            self._export_handoff(rid, tok)
        self.batcher.commit(plan, dec_tokens, pf_tokens)
        for rid, _ in handoff:                 # the decode side continues the request; it ends here
            self._vetoed[rid] = "handoff"
        for rid, toks in spec_extra.items():       # the accepted drafts beyond the first token, and the bonus token
            slot = self._slot_of.get(rid)
            for t in toks:
                if slot is not None:
                    self.req_table.advance(slot, int(t))
                self._observe(rid, int(t), now)
            self.batcher.commit_tokens(rid, [int(t) for t in toks])
        return self._collect()

    # ---- lockstep (data-parallel attention + expert parallelism) -----------------------------------
    def _agree(self, plan):
        import torch.distributed as dist
        f = torch.tensor([1 if plan.num_decode > 0 else 0, 1 if plan.num_prefill_seqs > 0 else 0, 1 if self.reqs else 0],
                         dtype=torch.int32, device=self.device)
        dist.all_reduce(f, op=dist.ReduceOp.MAX, group=self.lockstep)
        return [bool(x) for x in f.tolist()]

    def _empty_decode(self):
        """A decode forward with no live slot: this rank's experts still serve the other ranks' tokens."""
        ms = self.ms
        self.h_dec.zero_()
        self.h_dec[2 * ms:3 * ms] = -1          # no KV write
        self.d_dec.copy_(self.h_dec, non_blocking=self.device.type == "cuda")
        B = self._bucket(1)
        self._all_greedy = True
        if self.device.type == "cuda" and self.cfg.use_cuda_graphs and (B, True) in self.graphs:
            self.graphs[(B, True)].replay()
        else:
            self._decode_body(B)

    def _empty_prefill(self):
        dev = self.device
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        batch = ForwardBatch(token_ids=i32([0]), positions=i32([0]), slot_mapping=i32([-1]),
                             block_tables=torch.zeros((1, self.max_blocks), dtype=torch.int32, device=dev),
                             ctx_lens=i32([1]), is_decode=False, q_start=i32([0]), q_len=i32([1]), max_q_len=1)
        self._ep_bound(False)
        self.model.forward(batch, self.kv_caches, return_hidden=True)

    def precapture(self, buckets=None):
        """Capture the decode graphs up front. In lockstep mode every rank must call this with the same buckets:
        a capture's warm-up run executes the collective kernels, so it cannot happen on one rank alone later."""
        if self.device.type != "cuda" or not self.cfg.use_cuda_graphs:
            return
        if not self.reqs:        # nothing is running: capture on an empty step (no KV write, zero-length contexts)
            ms = self.ms
            self.h_dec.zero_()
            self.h_dec[2 * ms:3 * ms] = -1
            self.d_dec.copy_(self.h_dec, non_blocking=True)
        for B in (buckets or [b for b in DECODE_BUCKETS if b <= self.ms]):
            self._all_greedy = True
            if (B, True) not in self.graphs:
                self._capture(B)

    def _step_lockstep(self, plan) -> List[GenerateResult]:
        any_decode, any_prefill, any_work = self._agree(plan)
        self.global_has_work = any_work
        for it in plan.prefill:
            if it.start == 0 or self.slot_params[it.slot, 3] != float(it.seq_id):
                sp = self._params_of(it.seq_id)
                self.slot_params[it.slot] = (sp[0], sp[1], sp[2], float(it.seq_id))
                self._bind_slot(int(it.seq_id), int(it.slot))
        dec_tokens = np.zeros(self.ms, np.int32)
        pf_tokens = np.zeros(0, np.int32)
        if any_decode:
            if plan.num_decode > 0:
                dec_tokens = self._run_decode(plan).copy()
            else:
                self._empty_decode()
        if any_prefill:
            if plan.num_prefill_seqs > 0:
                pf_tokens = self._run_prefill(plan)
            else:
                self._empty_prefill()
        if plan.idle:
            return self._collect()
        self._check_device_status(plan)
        now = time.perf_counter()
        ids = plan.dec_seq_ids
        live = np.nonzero(ids >= 0)[0]
        self._count_decode(live, ids, dec_tokens, now)
        k = 0
        for it in plan.prefill:
            if it.last:
                self.req_table.advance(int(it.slot), int(pf_tokens[k]))
                self._observe(int(it.seq_id), int(pf_tokens[k]), now)
                k += 1
        self.batcher.commit(plan, dec_tokens, pf_tokens)
        return self._collect()

    def _params_of(self, rid):
        return self._req_params.get(rid, (0.0, 0, 1.0))

    def _bind_slot(self, rid: int, slot: int):
        """The per-slot request record (scheduler/request_state.py: 32 bytes per slot in pinned memory, the table a
        kernel or a monitoring thread can read) starts when a request's first prefill chunk gets its slot."""
        old = self._slot_of.get(rid)
        if old == slot:
            return
        generated = 0
        carried = (0, 0.0, 0.0)
        if old is not None and int(self.req_table.rec[old]["request_id"]) == rid:
            generated = int(self.req_table.rec[old]["generated"])      # a preempted request resumes in another slot
            carried = (int(self._sl_nout[old]), float(self._sl_tfirst[old]), float(self._sl_tlast[old]))
            self.req_table.release(old)
        self._slot_of[rid] = slot
        self._sl_nout[slot], self._sl_tfirst[slot], self._sl_tlast[slot] = carried
        st = self.reqs.get(rid)
        self._sl_slow[slot] = bool(st is not None and (st.hook is not None or st.stream is not None)) or rid in self._spec_idx
        p = self._req_limits.get(rid, (1 << 30, -1))
        self.req_table.assign(slot, rid, p[0], p[1])
        self.req_table.rec[slot]["generated"] = generated

    def request_states(self):
        """Snapshot of the live per-slot records (numpy structured array, one entry per slot)."""
        return self.req_table.rec.copy()

    def _count_decode(self, live, ids, dec_tokens, now: float):
        """One decode step's tokens: the per-slot record table and the token counters / timestamps as vector updates;
        only the slots of requests that asked for per-token work (hook, stream, draft index) go through ``_observe``."""
        self.req_table.advance_many(live, dec_tokens[live])
        bound = live[self.req_table.rec["request_id"][live] == ids[live].astype(np.uint64)]
        fresh = bound[self._sl_nout[bound] == 0]
        self._sl_tfirst[fresh] = now
        for sl in fresh:                      # first token produced by a decode step (a request imported after prefill)
            st = self.reqs.get(int(ids[sl]))
            if st is not None and not st.t_first:
                st.t_first = now
        self._sl_tlast[bound] = now
        self._sl_nout[bound] += 1
        slow = live[self._sl_slow[live]] if len(bound) == len(live) else live
        for sl in slow:
            self._observe(int(ids[sl]), int(dec_tokens[sl]), now, counted=bool(self._slot_of.get(int(ids[sl])) == sl))

    def _observe(self, rid: int, tok: int, now: float, counted: bool = False):
        st = self.reqs.get(rid)
        if st is None:
            return
        slot = self._slot_of.get(rid)
        if not counted:
            if slot is not None:
                if self._sl_nout[slot] == 0 and st.n_out == 0:
                    self._sl_tfirst[slot] = now
                    st.t_first = now          # time to first token is readable while the request still runs
                self._sl_tlast[slot] = now
                self._sl_nout[slot] += 1
            else:
                if st.n_out == 0:
                    st.t_first = now
                st.t_last = now
                st.n_out += 1
        idx = self._spec_idx.get(rid)
        if idx is not None:
            idx.extend([tok])
        if st.stream is not None:
            st.stream(rid, tok)
        if st.hook is not None:
            decision = st.hook(rid, tok, st.n_out + (int(self._sl_nout[slot]) if slot is not None else 0))
            if decision in ("veto", "terminate"):
                self._vetoed[rid] = decision
                if slot is not None:
                    from ..scheduler.request_state import ExitFlag
                    self.req_table.set_flag(slot, ExitFlag.VETO)

    def _collect(self) -> List[GenerateResult]:
        out = []
        vetoed = self._vetoed
        for rid in list(vetoed):
            self.batcher.abort(rid)
        for f in self.batcher.pop_finished():
            if self.kv_swap is not None:
                self.kv_swap.forget(f.id)
                self.kv_swap.drop(f.id)
            st = self.reqs.pop(f.id, None)
            self._sessions.discard(f.id)
            self.kv_importance.pop(f.id, None)
            slot = self._slot_of.pop(f.id, None)
            if slot is not None and int(self.req_table.rec[slot]["request_id"]) == f.id:
                if st is not None and self._sl_nout[slot]:      # fold the fast-path counters into the request's state
                    st.t_first = st.t_first or float(self._sl_tfirst[slot])
                    st.t_last = max(st.t_last, float(self._sl_tlast[slot]))
                    st.n_out += int(self._sl_nout[slot])
                self._sl_nout[slot] = 0
                self._sl_slow[slot] = False
                self.req_table.release(slot)
            self._req_limits.pop(f.id, None)
            self._req_params.pop(f.id, None)
            self._spec_idx.pop(f.id, None)
            self._mtp_cand.pop(f.id, None)
            self._eagle_feat.pop(f.id, None)
            toks = [int(t) for t in f.tokens]
            reason = S.FINISH_REASONS.get(f.finish, "length")
            if f.id in vetoed:
                how = vetoed.pop(f.id)
                reason = how
                if how == "veto" and toks:
                    toks = toks[:-1]  # the vetoed token is dropped
            tel = SequenceTelemetry(prompt_tokens=f.prompt_len, generated_tokens=len(toks),
                                    cached_prefix_tokens=f.cached_prefix, preemptions=f.preemptions)
            if st is not None:
                tel.ttft_ms = (st.t_first - st.t_submit) * 1e3 if st.t_first else 0.0
                tel.e2e_ms = (st.t_last - st.t_submit) * 1e3 if st.t_last else 0.0
                tel.tpot_ms = ((st.t_last - st.t_first) * 1e3 / max(st.n_out - 1, 1)) if st.n_out > 1 else 0.0
            text = self.tokenizer.decode(toks) if self.tokenizer is not None else ""
            r = GenerateResult(request_id=f.id, token_ids=toks, text=text, finish_reason=reason, telemetry=tel)
            METRICS.record_request(tel)
            self.results[f.id] = r
            out.append(r)
        return out

    # ------------------------------------------------------------------------------------------
    def run_until_done(self, max_steps: int = 10 ** 9) -> List[GenerateResult]:
        done = []
        steps = 0
        while steps < max_steps:
            plan_results = self.step()
            done.extend(plan_results)
            steps += 1
            if self.lockstep is not None:
                if not self.global_has_work:      # every rank of the group is drained
                    break
            elif not self.reqs:
                break
        return done

    def generate_batch(self, prompts: List[List[int]], *, max_tokens=256, temperature=0.7, top_k=0, top_p=1.0,
                       eos_ids=None) -> List[GenerateResult]:
        """All requests in one call; results come back in request order."""
        mt = max_tokens if isinstance(max_tokens, (list, tuple)) else [max_tokens] * len(prompts)
        ids = [self.submit(p, max_tokens=m, temperature=temperature, top_k=top_k, top_p=top_p, eos_ids=eos_ids)
               for p, m in zip(prompts, mt)]
        self.run_until_done()
        return [self.results.pop(i) for i in ids]
