"""CUDA-graph atlas over the shared KV history, on the B200 kernels.

Mirror of `bonsai_sft.gpu.fast_runtime` (src/bonsai_sft/gpu/fast_runtime.py:58-561):
`GraphAtlas` keeps one KV buffer per capacity segment sigma, shared by every replay
width and role, captures one CUDA graph per (M, sigma, role) and exposes the same
per-step calls (`get_graph`, `prepare_step`, `commit_kv`, `commit_kv_from_verify`,
`migrate_segment`, `select_segment`).

What differs from the reference, by design:
  * a captured graph holds only hand-written kernels (about ten per layer);
  * visibility is computed inside the attention kernel from a 16-byte device record, so
    `prepare_step` is one tiny launch instead of a mask copy plus slice fills, and
    `CapturedGraph.attn_mask` is that record (int32 [4]: cache_len, n_pend, role, P);
  * attention reads history rows [0, cache_len) only, so the cost of a replay does not
    grow with the segment size;
  * intermediates live in one workspace per width, so capturing a role or a segment
    more costs no activation memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import native, ops
from .contracts import validate_graph_roles
from .model import PREFILL_CHUNK, ModelArgs, SDLMLayerCache, Transformer, make_sdlm_cache

DEFAULT_SEGMENT_LADDER = (256, 1024, 4096)
DEFAULT_M_SET = (1, 8, 9, 10, 12, 16, 17)
ROLES = ("draft", "verify", "ar")

# head of each role (fast_runtime.py:179-205): native packed T2 everywhere, the dense e4m3 / bf16 tied
# table for the acceptance-tolerant draft variants
ROLE_HEAD_PRECISION = {"ar": "t2", "draft": "t2", "verify": "t2", "draft_fp8": "fp8", "draft_bf16": "bf16_raw"}

_ROLE_ID = {"draft": native.ROLE_DRAFT, "draft_fp8": native.ROLE_DRAFT,
            "draft_bf16": native.ROLE_DRAFT, "verify": native.ROLE_VERIFY, "ar": native.ROLE_AR}


@dataclass
class CapturedGraph:
    """Same fields as the reference's record (fast_runtime.py:58-73)."""
    cuda_graph: "torch.cuda.CUDAGraph"
    tokens_buf: torch.Tensor              # int64 [M]
    positions_buf: torch.Tensor           # int64 [M]
    attn_mask: torch.Tensor               # int32 [4] step record (see module docstring)
    logits_out: torch.Tensor              # fp32 [logits_end-logits_start, vocab]
    kv_full: List[SDLMLayerCache]         # views into the shared per-sigma buffer
    M: int
    sigma: int
    role: str
    P: int
    logits_start: int
    logits_end: int
    lm_head_precision: str
    flex_attn_fn: Optional[object] = None  # kept for field compatibility; always None
    n_kernels: int = 0                     # this library's kernel nodes in the graph (bm_launch_count at capture)


def role_logit_rows(role: str, M: int, D: int) -> Tuple[int, int]:
    """Logit rows a role needs (fast_runtime.py:179-205): ar -> the one row; draft ->
    the D block rows; verify -> the anchor row and the D draft rows."""
    P = M - D
    if role == "ar":
        return 0, M
    if role in ("draft", "draft_fp8", "draft_bf16"):
        return P, M
    if role == "verify":
        return 0, min(D + 1, M)
    raise ValueError(f"unsupported graph role: {role!r}")


class GraphAtlas:
    """Pre-captured CUDA graphs keyed by (M, sigma, role)."""

    def __init__(self, model: Transformer, args: ModelArgs, device, dtype: torch.dtype = torch.bfloat16,
                 segment_ladder: Tuple[int, ...] = DEFAULT_SEGMENT_LADDER,
                 m_set: Tuple[int, ...] = DEFAULT_M_SET, roles: Tuple[str, ...] = ROLES,
                 capture_verbose: bool = True, use_flex_attention: bool = True):
        self.model = model
        self.args = args
        self.device = torch.device(device)
        self.dtype = dtype
        self.segment_ladder = tuple(sorted(set(segment_ladder)))
        self.m_set = tuple(sorted(set(m_set)))
        self.roles = tuple(roles)
        validate_graph_roles(self.roles)
        self.D = args.block_size
        self.M_max = max(self.m_set)
        self.vocab_size = args.vocab_size
        self.n_layers = args.n_layers
        self.n_kv = args.n_kv_heads
        self.head_dim = args.head_dim
        self.use_flex_attention = False      # accepted for signature compatibility
        if capture_verbose:
            print(f"[GraphAtlas] D={self.D}, segments={self.segment_ladder}, M_set={self.m_set}, "
                  f"roles={self.roles}, kernels={native.lib().bm_version().decode()}")
        self.model.prepare_t2_lm_head()
        if "draft_fp8" in self.roles:                  # fast_runtime.py:112-114
            self.model.prepare_fp8_lm_head()
        if "draft_bf16" in self.roles:
            self.model.prepare_bf16_lm_head()
        self._allocate_shared_kv()
        self._allocate_input_bufs()
        self._capture_all()

    # ------------------------------------------------------------------ allocation
    def _allocate_shared_kv(self) -> None:
        """One [2, L, 1, n_kv, sigma + M_max, hd] buffer per sigma (fast_runtime.py:130-138)
        and the attention scratch that goes with it."""
        self.kv_buffers: Dict[int, torch.Tensor] = {}
        self.attn_scratch: Dict[int, torch.Tensor] = {}
        for sigma in self.segment_ladder:
            self.kv_buffers[sigma] = torch.zeros(
                2, self.n_layers, 1, self.n_kv, sigma + self.M_max, self.head_dim,
                device=self.device, dtype=self.dtype)
            self.attn_scratch[sigma] = ops.attention_scratch(self.M_max, self.args.n_heads, sigma,
                                                             self.device)

    def _allocate_input_bufs(self) -> None:
        """int64 token / position buffers per width (fast_runtime.py:144-149)."""
        self.tokens_m: Dict[int, torch.Tensor] = {}
        self.positions_m: Dict[int, torch.Tensor] = {}
        for M in self.m_set:
            self.tokens_m[M] = torch.zeros(M, device=self.device, dtype=torch.int64)
            self.positions_m[M] = torch.zeros(M, device=self.device, dtype=torch.int64)

    # ------------------------------------------------------------------ capture
    def _capture_all(self) -> None:
        """M = 1 captures the 'ar' role only; wider graphs capture every other requested
        role (fast_runtime.py:154-169)."""
        self.graphs: Dict[Tuple[int, int, str], CapturedGraph] = {}
        for sigma in self.segment_ladder:
            for M in self.m_set:
                if M == 1:
                    if "ar" in self.roles:
                        self.graphs[(M, sigma, "ar")] = self._capture_one(M, sigma, "ar")
                    continue
                for role in self.roles:
                    if role != "ar":
                        self.graphs[(M, sigma, role)] = self._capture_one(M, sigma, role)
        # Prompt slabs: one AR-causal graph of PREFILL_CHUNK rows per segment, layers only (the one
        # logit row a prompt needs is taken afterwards).  Kept apart from `graphs`, whose key set
        # mirrors the reference's.  Needs workspace rows for a whole slab.
        self.prefill_graphs: Dict[int, CapturedGraph] = {}
        if self.M_max >= PREFILL_CHUNK:
            self.prefill_tokens = torch.zeros(PREFILL_CHUNK, device=self.device, dtype=torch.int64)
            self.prefill_positions = torch.zeros(PREFILL_CHUNK, device=self.device, dtype=torch.int64)
            self.prefill_logits = torch.zeros((1, self.model.workspace(PREFILL_CHUNK).n_pad),
                                              dtype=torch.float32, device=self.device)
            for sigma in self.segment_ladder:
                self.prefill_graphs[sigma] = self._capture_one(
                    PREFILL_CHUNK, sigma, "ar", logit_rows=(0, 0),
                    buffers=(self.prefill_tokens, self.prefill_positions))

    def _capture_one(self, M: int, sigma: int, role: str, logit_rows: Optional[Tuple[int, int]] = None,
                     buffers: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> CapturedGraph:
        D = self.D
        P = M - D
        ls, le = logit_rows if logit_rows is not None else role_logit_rows(role, M, D)
        precision = ROLE_HEAD_PRECISION[role]
        shared = self.kv_buffers[sigma]
        slot = shared[:, :, :, :, : sigma + M, :]
        kv_full = [(slot[0, i], slot[1, i]) for i in range(self.n_layers)]
        state = ops.new_step_state(self.device)
        ops.set_step_state(state, 0, 0, _ROLE_ID[role], P)
        tokens_buf, positions_buf = buffers if buffers is not None else (self.tokens_m[M], self.positions_m[M])
        ws = self.model.workspace(M)
        logits_buf = torch.zeros((le - ls, ws.n_pad), dtype=torch.float32, device=self.device)
        scratch = self.attn_scratch[sigma]

        def body():
            return self.model.forward_sdlm_decode_graph_kernel(
                token_values=tokens_buf, positions=positions_buf, kv_full=kv_full, block_size=M,
                attn_mask=state, logits_start=ls, logits_end=le, lm_head_precision=precision,
                attn_scratch=scratch, logits_buf=logits_buf, stable_state=True)

        # One eager pass on a side stream (sets kernel attributes, proves the launch
        # sequence), then capture.
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            body()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        launches_before = native.lib().bm_launch_count()
        with torch.cuda.graph(graph):
            logits = body()
        n_kernels = int(native.lib().bm_launch_count() - launches_before)
        return CapturedGraph(cuda_graph=graph, tokens_buf=tokens_buf, positions_buf=positions_buf,
                             attn_mask=state, logits_out=logits, kv_full=kv_full, M=M, sigma=sigma,
                             role=role, P=P, logits_start=ls, logits_end=le, lm_head_precision=precision,
                             n_kernels=n_kernels)

    # ------------------------------------------------------------------ selection
    def select_segment(self, needed_kv_len: int) -> int:
        """Smallest sigma in the ladder >= needed_kv_len, else the largest
        (fast_runtime.py:377-386)."""
        for sigma in self.segment_ladder:
            if needed_kv_len <= sigma:
                return sigma
        return self.segment_ladder[-1]

    def get_graph(self, M: int, sigma: int, role: str, cache_len: Optional[int] = None) -> CapturedGraph:
        """The graph of (M, sigma, role).  `cache_len` is accepted for callers that know the history length;
        one graph serves every length."""
        return self.graphs[(M, sigma, role)]

    # ------------------------------------------------------------------ per-step API
    def prepare_step(self, graph: CapturedGraph, cache_len: int, n_pend: int,
                     causal_attn: bool = True) -> None:
        """Tell the graph's attention what is visible in this replay: draft -> block-causal
        SDLM visibility over `n_pend` pending rows; verify -> AR-causal with the repeated
        history anchor hidden; ar -> AR-causal (fast_runtime.py:391-465)."""
        if graph.role == "verify" and cache_len <= 0:
            raise RuntimeError("batched verifier requires a committed anchor")
        n_pend_clamp = max(0, min(int(n_pend), max(graph.P, 0)))
        ops.set_step_state(graph.attn_mask, int(cache_len), n_pend_clamp, _ROLE_ID[graph.role], graph.P)

    # One launch instead of the tensor fills + prepare_step of a step.  The decode loops use these for
    # graphs whose buffers live on the GPU (a CPU stand-in atlas for host-logic tests keeps the fills).
    def stage_draft(self, graph: CapturedGraph, pending: torch.Tensor, n_pend: int, cache_len: int, D: int,
                    mask_id: int) -> None:
        ops.stage_replay_inputs(0, pending, None, n_pend, cache_len, graph.M, D, mask_id, _ROLE_ID[graph.role],
                                graph.P, graph.tokens_buf, graph.positions_buf, graph.attn_mask)

    def stage_draft_after_commit(self, graph: CapturedGraph, src: torch.Tensor, n_commit: int, verified: bool,
                                 gen_dst: torch.Tensor, pending: torch.Tensor, cache_len: int, D: int,
                                 mask_id: int) -> None:
        """The previous step's commit (ids -> output buffer and pending rows) and this draft replay's inputs in
        one launch."""
        ops.commit_stage_draft(src, n_commit, verified, gen_dst, pending,
                               stage=(cache_len, graph.M, D, mask_id, _ROLE_ID[graph.role], graph.P,
                                      graph.tokens_buf, graph.positions_buf, graph.attn_mask))

    def stage_verify(self, graph: CapturedGraph, pending: torch.Tensor, n_pend: int, draft_tokens: torch.Tensor,
                     cache_len: int, D: int) -> None:
        if cache_len <= 0:
            raise RuntimeError("batched verifier requires a committed anchor")
        ops.stage_replay_inputs(1, pending, draft_tokens, n_pend, cache_len, graph.M, D, 0, _ROLE_ID[graph.role],
                                graph.P, graph.tokens_buf, graph.positions_buf, graph.attn_mask)

    def stage_ar(self, graph: CapturedGraph, token: torch.Tensor, position: int) -> None:
        ops.stage_replay_inputs(2, token, None, 0, position, 1, 0, 0, _ROLE_ID[graph.role], graph.P,
                                graph.tokens_buf, graph.positions_buf, graph.attn_mask)

    def commit_kv(self, graph: CapturedGraph, cache_len: int, n_accept: int) -> None:
        """Rows [sigma, sigma+n_accept) -> history rows [cache_len, cache_len+n_accept) in
        every layer of the segment's buffer (fast_runtime.py:467-484)."""
        if n_accept <= 0:
            return
        sigma = graph.sigma
        ops.kv_copy_rows(self.kv_buffers[sigma], sigma + self.M_max, sigma, cache_len, n_accept)

    def commit_kv_from_verify(self, verify_graph: CapturedGraph, cache_len: int, n_accept: int) -> None:
        """Promote the verifier's rows of the accepted draft tokens, which sit one past the
        repeated anchor: [sigma+1, sigma+1+n_accept) -> [cache_len, ...)
        (fast_runtime.py:486-508)."""
        if n_accept <= 0:
            return
        sigma = verify_graph.sigma
        ops.kv_copy_rows(self.kv_buffers[sigma], sigma + self.M_max, sigma + 1, cache_len, n_accept)

    def prefill(self, prompt_ids: torch.Tensor, sigma: int) -> torch.Tensor:
        """The prompt's K/V into history rows [0, len) of segment `sigma`, by replaying the captured
        slab graph once per PREFILL_CHUNK rows (staging, replay, row promotion: three launches + one
        graph per slab), then the last row's logits through the packed head.  Same arithmetic as
        Transformer.forward_sdlm_prefill, which launches every operator of every slab from the host
        and computes all rows' logits; the decode loops need only the last row (reference:
        fast_generate.py:203-222 take `logits[-1]`).  Returns fp32 logits [1, vocab]."""
        seq = int(prompt_ids.shape[0])
        if seq < 1 or seq > sigma:
            raise ValueError(f"prompt of {seq} tokens does not fit segment {sigma}")
        if self.model.wide_prefill_supported() and seq > PREFILL_CHUNK:
            # the many-row kernels: every projection reads its weights once per 32 prompt rows, one
            # attention launch per layer; K / V rows land in place.  Bit-identical to the slab replays below.
            shared = self.kv_buffers[sigma]
            planes = [(shared[0, i], shared[1, i]) for i in range(self.n_layers)]
            return self.model.prefill_wide(prompt_ids, planes, sigma + self.M_max, self.prefill_logits
                                           if getattr(self, "prefill_logits", None) is not None else None)
        g = self.prefill_graphs[sigma]
        ids = prompt_ids.to(torch.int64).contiguous()
        n = 0
        for c0 in range(0, seq, PREFILL_CHUNK):
            n = min(PREFILL_CHUNK, seq - c0)
            ops.stage_replay_inputs(3, ids[c0:], None, n, c0, PREFILL_CHUNK, self.D, 0, native.ROLE_AR, g.P,
                                    g.tokens_buf, g.positions_buf, g.attn_mask)
            g.cuda_graph.replay()
            ops.kv_copy_rows(self.kv_buffers[sigma], sigma + self.M_max, sigma, c0, n)
        return self.model.head_from_workspace(PREFILL_CHUNK, n - 1, 1, self.prefill_logits)

    def migrate_segment(self, src_sigma: int, dst_sigma: int, cache_len: int) -> None:
        """Copy live rows [0, cache_len) into a larger segment (fast_runtime.py:510-521)."""
        if src_sigma == dst_sigma:
            return
        src, dst = self.kv_buffers[src_sigma], self.kv_buffers[dst_sigma]
        dst[:, :, :, :, :cache_len, :].copy_(src[:, :, :, :, :cache_len, :])


def prefill_to_atlas(model: Transformer, atlas: GraphAtlas, prompt_ids: torch.Tensor,
                     target_sigma: int, fast: bool = False, causal_attn: bool = True) -> int:
    """Prefill once and place the prompt's K/V in the target segment
    (fast_runtime.py:530-561).  Returns the new cache_len."""
    seq_len = prompt_ids.shape[0]
    cache = make_sdlm_cache(model.args, device=atlas.device)
    model.forward_sdlm_prefill(token_values=prompt_ids, cache=cache,
                               positions=torch.arange(seq_len, device=atlas.device),
                               block_size=1, fast=fast, causal_attn=causal_attn)
    shared = atlas.kv_buffers[target_sigma]
    for i, (ck, cv) in enumerate(cache):
        shared[0, i, :, :, :seq_len, :].copy_(ck[0])
        shared[1, i, :, :, :seq_len, :].copy_(cv[0])
    return seq_len
