"""Decode policies over the GraphAtlas: AR, confidence, speculative and hybrid.

Mirror of `bonsai_sft.gpu.fast_generate` (src/bonsai_sft/gpu/fast_generate.py): the same
four entry points with the same arguments, token semantics and statistics dictionary.
The step mechanics shared by the loops (prefill + first token, segment choice and
migration, draft and verifier replays with their input rows, KV promotion) live in
`_Session`; each policy is then a short loop.  Argmax, the confidence chain and the
prefix-accept count are native kernels (`ops.argmax_rows`, `ops.draft_chain`,
`ops.verify_accept`).

Input rows of a draft replay of width M = P + D with n_pend pending tokens
(fast_generate.py:1016-1027):
    tokens     [pending(n_pend) | PAD=0 (P-n_pend) | anchor=pending[-1] | MASK x (D-1)]
    positions  [cache_len .. cache_len+n_pend) | 0 ... | cache_len+n_pend-1 .. +D-1]
and of a verifier replay of width D+1 (fast_generate.py:1044-1050):
    tokens     [anchor | draft[0..D)]          positions  cache_len-1 .. cache_len+D-1
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import ops
from .contracts import validate_native_verifier, validate_verification_options
from .fast_runtime import CapturedGraph, GraphAtlas
from .model import Transformer, make_sdlm_cache

_BONSAI_EOS_IDS = frozenset([151643, 151645])  # <|endoftext|>, <|im_end|>


# --------------------------------------------------------------------------- small helpers
def _first_stop_index(text: str, stop_strings: Optional[Sequence[str]]) -> int:
    """Earliest character index of any stop string, len(text) if none occurs."""
    hits = [text.find(s) for s in (stop_strings or ()) if s]
    hits = [h for h in hits if h != -1]
    return min(hits) if hits else len(text)


def _decode_hits_stop(tokenizer, token_ids: Sequence[int], stop_strings) -> bool:
    if not stop_strings or not token_ids:
        return False
    text = tokenizer.decode(list(token_ids), skip_special_tokens=True)
    return _first_stop_index(text, stop_strings) < len(text)


def _argmax_rows(logits: torch.Tensor, out=None) -> torch.Tensor:
    """Row argmax, lowest index on ties (native kernel); written into `out` when given.  `out` may be
    (tensor, scratch): with the scratch of ops.logit_scratch every row is reduced by 16-128 CTAs."""
    if isinstance(out, tuple):
        return ops.argmax_rows(logits, out=out[0], scratch=out[1])
    return ops.argmax_rows(logits, out=out)


def _fused_draft_chain(logits: torch.Tensor, threshold: float,
                       out: Optional[Tuple[torch.Tensor, ...]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(draft ids [D], iter_accept) with iter_accept = 1 + the number of leading rows
    r >= 1 whose confidence exp(max - logsumexp) exceeds the threshold
    (fast_generate.py:111-130).  Row 0 is always committed.  `out` = (ids, max work area,
    confidences, count[, scratch]) places the results in the caller's buffers; with the scratch of
    ops.logit_scratch the reductions run on 16-128 CTAs per row."""
    if out is not None and len(out) > 4:
        idx, n, _ = ops.draft_chain(logits, threshold, bufs=tuple(out[:4]), scratch=out[4])
    else:
        idx, n, _ = ops.draft_chain(logits, threshold, bufs=out)
    return idx, n


def _fused_verify_accept(draft_tokens: torch.Tensor, verify_tokens: torch.Tensor, D: int,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Length of the longest prefix of identical token ids (fast_generate.py:133-146);
    logits are deliberately not an input."""
    return ops.verify_accept(draft_tokens, verify_tokens, D, out=out)


def _read_record(rec: torch.Tensor, *parts: torch.Tensor) -> List[List[int]]:
    """Host copies of `parts` as lists.  When the parts tile the front of `rec` in order
    (the decode buffers are laid out that way) this is ONE device-to-host copy and one
    synchronisation; otherwise one per part."""
    addr, total = rec.data_ptr(), 0
    tiled = rec.is_contiguous()
    for p in parts:
        tiled = (tiled and p.dtype == rec.dtype and p.is_contiguous()
                 and p.data_ptr() == addr + total * rec.element_size())
        total += p.numel()
    if not tiled or total > rec.numel():
        return [p.reshape(-1).tolist() for p in parts]
    flat = rec[:total].tolist()
    out, at = [], 0
    for p in parts:
        out.append(flat[at:at + p.numel()])
        at += p.numel()
    return out


_PINNED: dict = {}          # host staging buffers for _begin_read, by element count (pinned once, reused)


def _begin_read(rec: torch.Tensor, *parts: torch.Tensor):
    """Start the device-to-host copy of `parts` (see _read_record) without waiting for it: the copy goes to a
    pinned buffer behind an event, so launches queued after this call overlap the host's wait.  Returns a
    handle for _finish_read.  CPU tensors, or parts that do not tile the record, are read at once."""
    addr, total = rec.data_ptr(), 0
    tiled = rec.is_contiguous() and rec.is_cuda
    for p in parts:
        tiled = (tiled and p.dtype == rec.dtype and p.is_contiguous()
                 and p.data_ptr() == addr + total * rec.element_size())
        total += p.numel()
    if not tiled or total > rec.numel():
        return (None, None, _read_record(rec, *parts))
    key = (rec.dtype, total)
    slot = _PINNED.get(key)
    if slot is None:
        slot = _PINNED[key] = (torch.empty(total, dtype=rec.dtype).pin_memory(), torch.cuda.Event())
    host, event = slot
    host.copy_(rec[:total], non_blocking=True)
    event.record()
    return (host, event, [p.numel() for p in parts])


def _finish_read(handle) -> List[List[int]]:
    host, event, sizes = handle
    if host is None:
        return sizes
    event.synchronize()
    flat = host.tolist()
    out, at = [], 0
    for n in sizes:
        out.append(flat[at:at + n])
        at += n
    return out


def _select_M_for_pending(atlas, n_pend: int) -> int:
    """Smallest captured width with room for n_pend pending rows ahead of the D block rows
    (fast_generate.py:574-583).  D=8, widths {9,10,12,16,17}: 1->9, 2->10, 3-4->12,
    5-8->16, 9->17."""
    for M in atlas.m_set:
        if M - atlas.D >= n_pend and M >= n_pend + atlas.D:
            return M
    return atlas.m_set[-1]


def _draft_role(atlas, use_fp8: bool, use_bf16: bool = False) -> str:
    """fast_generate.py:586-599."""
    if use_fp8 and use_bf16:
        raise RuntimeError("FP8 and BF16 draft roles are mutually exclusive")
    role = "draft_fp8" if use_fp8 else ("draft_bf16" if use_bf16 else "draft")
    if role not in atlas.roles:
        raise RuntimeError(f"requested draft role was not captured: {role}")
    return role


def _verify_role(atlas, use_fp8: bool = False, use_q1: bool = False, use_w1a16: bool = False) -> str:
    """fast_generate.py:602-608."""
    validate_native_verifier(use_fp8, use_q1, use_w1a16)
    if "verify" not in atlas.roles:
        raise RuntimeError("requested native verify role was not captured")
    return "verify"


@dataclass
class _DecodeBufs:
    """Device buffers that live for one generate call (fast_generate.py:69-104)."""
    gen_buf: torch.Tensor       # int64 [max_gen_len + M_max + 1]
    pending_buf: torch.Tensor   # int64 [M_max + 1]
    commit_buf: torch.Tensor    # int64 [M_max + 1]
    pos_arange: torch.Tensor    # int64 [max(M_max + 1, prompt_len)]
    has_eos: bool
    M_max: int
    # Result records, each read by the host in one copy.  The count slots are int64 words whose
    # low half the kernels write as int32 (the high half stays zero).
    chain_rec: torch.Tensor     # int64 [D + 1]: draft ids | confidence-chain length
    chain_work: torch.Tensor    # fp32 [2, D]: row maxima and confidences of the chain kernel
    verify_rec: torch.Tensor    # int64 [2D + 2]: verifier ids (D + 1) | accepted count | draft ids (D)

    logit_scratch: Optional[torch.Tensor] = None   # ops.logit_scratch: partials of the many-CTA logit reductions

    def chain_out(self, D: int):
        out = (self.chain_rec[:D], self.chain_work[0], self.chain_work[1], self.chain_rec[D:D + 1])
        return out + (self.logit_scratch,) if self.logit_scratch is not None else out

    def argmax_out(self, view: torch.Tensor):
        return (view, self.logit_scratch) if self.logit_scratch is not None else view


def _alloc_decode_bufs(atlas, max_gen_len: int, eos_ids, prompt_len: int = 0) -> _DecodeBufs:
    dev = atlas.device
    m_max = max(atlas.M_max, 1)
    D = max(int(atlas.D), 1)
    return _DecodeBufs(
        chain_rec=torch.zeros(D + 1, dtype=torch.long, device=dev),
        chain_work=torch.zeros((2, D), dtype=torch.float32, device=dev),
        verify_rec=torch.zeros(2 * D + 2, dtype=torch.long, device=dev),
        logit_scratch=ops.logit_scratch(dev) if torch.device(dev).type == "cuda" else None,
        gen_buf=torch.zeros(max_gen_len + m_max + 1, dtype=torch.long, device=dev),
        pending_buf=torch.zeros(m_max + 1, dtype=torch.long, device=dev),
        commit_buf=torch.zeros(m_max + 1, dtype=torch.long, device=dev),
        pos_arange=torch.arange(max(m_max + 1, prompt_len), dtype=torch.long, device=dev),
        has_eos=bool(eos_ids), M_max=m_max)


def _commit_and_eos(bufs: _DecodeBufs, n_commit: int, eos_set,
                    host_tokens: Optional[List[int]] = None) -> Tuple[List[int], bool, int]:
    """Host scan of the committed ids for EOS; the EOS token itself is not kept
    (fast_generate.py:149-171).  The ids come from `host_tokens` when the caller has already
    read them, else from one bulk device-to-host copy of commit_buf."""
    if n_commit <= 0:
        return [], False, 0
    toks = host_tokens[:n_commit] if host_tokens is not None else bufs.commit_buf[:n_commit].tolist()
    if not eos_set:
        return toks, False, n_commit
    for kept, t in enumerate(toks):
        if t in eos_set:
            return toks, True, kept
    return toks, False, n_commit


# --------------------------------------------------------------------------- session mechanics
class _Session:
    """State and step mechanics shared by the decode loops of one generate call."""

    def __init__(self, model: Transformer, atlas: GraphAtlas, input_ids: torch.Tensor,
                 max_gen_len: int, eos_ids):
        self.model, self.atlas = model, atlas
        self.args = model.args
        self.device = atlas.device
        self.D = self.args.block_size
        self.MASK = self.args.mask_token_id
        self.eos_ids = eos_ids
        self.max_gen_len = max_gen_len
        self.prompt_ids = input_ids[0].to(self.device)
        self.seq_len = int(self.prompt_ids.shape[0])
        self.bufs = _alloc_decode_bufs(atlas, max_gen_len, eos_ids, prompt_len=self.seq_len)
        self.cache_len = 0
        self.sigma = atlas.segment_ladder[0]
        self._deferred = None        # (ids, count, verified, output offset) of a commit not yet written

    # -- prefill, first token, segment choice (fast_generate.py:203-222, 951-969)
    def start(self) -> Tuple[float, int, float]:
        """Returns (prefill_time, first_token, t0).  The first token is the greedy argmax of
        the prompt's last row; the prompt's K/V is placed in the chosen segment."""
        atlas, bufs = self.atlas, self.bufs
        t0 = time.time()
        self.sigma = atlas.select_segment(self.seq_len + self.max_gen_len + atlas.M_max)
        shared = atlas.kv_buffers[self.sigma]
        shared.zero_()
        if getattr(atlas, "prefill_graphs", None) and self.seq_len <= self.sigma:
            # captured slab graphs write the prompt's rows straight into the segment
            logits = atlas.prefill(self.prompt_ids, self.sigma)
        else:
            cache = make_sdlm_cache(self.args, device=self.device)
            logits = self.model.forward_sdlm_prefill(
                token_values=self.prompt_ids, cache=cache, positions=bufs.pos_arange[: self.seq_len],
                block_size=1, fast=False, causal_attn=True)
            for i, (ck, cv) in enumerate(cache):
                shared[0, i, :, :, : self.seq_len, :].copy_(ck[0])
                shared[1, i, :, :, : self.seq_len, :].copy_(cv[0])
            del cache
        first = _argmax_rows(logits[-1:].contiguous(), bufs.argmax_out(bufs.gen_buf[0:1]))
        if first.data_ptr() != bufs.gen_buf.data_ptr():
            bufs.gen_buf[0:1].copy_(first)
        self.cache_len = self.seq_len
        torch.cuda.synchronize()
        prefill_time = time.time() - t0
        return prefill_time, int(bufs.gen_buf[0].item()), t0

    def ensure_room(self) -> None:
        """Move to a larger segment before the workspace rows would run past this one
        (fast_generate.py:1009-1013)."""
        atlas = self.atlas
        if self.cache_len + atlas.M_max > self.sigma:
            new_sigma = atlas.select_segment(self.cache_len + atlas.M_max + 64)
            if new_sigma != self.sigma:
                atlas.migrate_segment(self.sigma, new_sigma, self.cache_len)
                self.sigma = new_sigma

    def out_of_room(self, n_pend: int) -> bool:
        return self.cache_len + n_pend + self.D > self.atlas.segment_ladder[-1]

    # -- one AR replay (fast_generate.py:247-256)
    def ar_step(self, token, position: int) -> CapturedGraph:
        atlas = self.atlas
        g = atlas.get_graph(1, self.sigma, "ar")
        if isinstance(token, torch.Tensor) and token.dtype == torch.int64 and g.tokens_buf.is_cuda:
            atlas.stage_ar(g, token.reshape(1), position)      # token, position and step record in one launch
        else:
            if isinstance(token, torch.Tensor):
                g.tokens_buf[0:1].copy_(token.reshape(1))
            else:
                g.tokens_buf[0] = int(token)
            g.positions_buf[0] = position
            atlas.prepare_step(g, position, n_pend=0)
        g.cuda_graph.replay()
        atlas.commit_kv(g, position, n_accept=1)
        return g

    # -- commit of a step: ids -> output buffer and pending rows (fast_generate.py:1121-1140).  Deferred so
    #    that the next draft replay's staging kernel can do it in the same launch.
    @staticmethod
    def _device_ids(t: torch.Tensor) -> bool:
        return t.is_cuda and t.dtype == torch.int64 and t.is_contiguous()

    def defer_commit(self, src: torch.Tensor, n_commit: int, verified: bool, gen_off: int) -> None:
        self.flush_commit()
        self._deferred = (src, int(n_commit), bool(verified), int(gen_off))

    def flush_commit(self) -> None:
        d, self._deferred = self._deferred, None
        if d is None:
            return
        src, n, verified, off = d
        bufs = self.bufs
        if self._device_ids(src):
            ops.commit_stage_draft(src, n, verified, bufs.gen_buf[off:], bufs.pending_buf)
            return
        bufs.gen_buf[off:off + n].copy_(src[:n])
        if verified:
            bufs.pending_buf[0:1].copy_(src[n - 1:n])
        else:
            bufs.pending_buf[:n].copy_(src[:n])

    # -- draft replay: materialises the pending rows, proposes D tokens
    def draft_step(self, n_pend: int, role: str) -> CapturedGraph:
        atlas, bufs, D = self.atlas, self.bufs, self.D
        M = _select_M_for_pending(atlas, n_pend)
        P = M - D
        self.ensure_room()
        g = atlas.get_graph(M, self.sigma, role, self.cache_len)
        d = self._deferred
        if (d is not None and g.tokens_buf.is_cuda and self._device_ids(d[0]) and 1 <= n_pend <= P
                and n_pend == (1 if d[2] else d[1])):
            # the previous step's commit and this replay's inputs in one launch
            self._deferred = None
            atlas.stage_draft_after_commit(g, d[0], d[1], d[2], bufs.gen_buf[d[3]:], bufs.pending_buf,
                                           self.cache_len, D, self.MASK)
            g.cuda_graph.replay()
            atlas.commit_kv(g, self.cache_len, n_pend)
            self.cache_len += n_pend
            return g
        self.flush_commit()
        if g.tokens_buf.is_cuda and 1 <= n_pend <= P:
            atlas.stage_draft(g, bufs.pending_buf, n_pend, self.cache_len, D, self.MASK)
            g.cuda_graph.replay()
            atlas.commit_kv(g, self.cache_len, n_pend)
            self.cache_len += n_pend
            return g
        tok, pos = g.tokens_buf, g.positions_buf
        tok[:n_pend].copy_(bufs.pending_buf[:n_pend])
        if n_pend < P:
            tok[n_pend:P].zero_()
            pos[n_pend:P].zero_()
        # the block's anchor: the last pending token, or, for a block with nothing pending (the first block of the
        # confidence policy), the last history token, which the caller left in pending_buf[0]
        tok[P:P + 1].copy_(bufs.pending_buf[n_pend - 1:n_pend] if n_pend > 0 else bufs.pending_buf[0:1])
        if P + 1 < M:
            tok[P + 1:].fill_(self.MASK)
        torch.add(bufs.pos_arange[:n_pend], self.cache_len, out=pos[:n_pend])
        torch.add(bufs.pos_arange[:D], self.cache_len + n_pend - 1, out=pos[P:P + D])
        atlas.prepare_step(g, self.cache_len, n_pend=n_pend)
        g.cuda_graph.replay()
        atlas.commit_kv(g, self.cache_len, n_pend)
        self.cache_len += n_pend
        return g

    # -- width-(D+1) verifier inputs and replay
    def stage_verify(self, n_pend: int, draft_tokens: torch.Tensor, role: str) -> CapturedGraph:
        atlas, bufs, D = self.atlas, self.bufs, self.D
        gv = atlas.get_graph(D + 1, self.sigma, role, self.cache_len)
        if gv.tokens_buf.is_cuda and draft_tokens.dtype == torch.int64 and draft_tokens.is_contiguous():
            atlas.stage_verify(gv, bufs.pending_buf, n_pend, draft_tokens, self.cache_len, D)
            return gv
        gv.tokens_buf[0:1].copy_(bufs.pending_buf[n_pend - 1:n_pend])
        gv.tokens_buf[1:1 + D].copy_(draft_tokens)
        torch.add(bufs.pos_arange[:D + 1], self.cache_len - 1, out=gv.positions_buf[:D + 1])
        atlas.prepare_step(gv, self.cache_len, n_pend=0)
        return gv

    def verify_and_commit(self, gv: CapturedGraph, draft_tokens: torch.Tensor,
                          draft_host: Optional[List[int]] = None) -> Tuple[int, List[int]]:
        """Replay the verifier, accept the longest matching prefix, build
        commit_buf = draft[:acc] | verify[acc], promote the accepted rows.  Returns
        (acc, the acc + 1 committed ids on the host).  The verifier's ids, the count and (when
        the caller has not read them yet) the draft ids come back in one host read."""
        atlas, bufs, D = self.atlas, self.bufs, self.D
        gv.cuda_graph.replay()
        rec = bufs.verify_rec
        verify_tokens = _argmax_rows(gv.logits_out, bufs.argmax_out(rec[:D + 1]))
        acc_t = _fused_verify_accept(draft_tokens, verify_tokens, D, rec[D + 1:D + 2])
        if draft_host is None:
            verify_host, acc_host, draft_host = _read_record(rec, verify_tokens, acc_t, draft_tokens)
        else:
            verify_host, acc_host = _read_record(rec, verify_tokens, acc_t)
        acc = int(acc_host[0])
        if acc > 0:
            bufs.commit_buf[:acc].copy_(draft_tokens[:acc])
        bufs.commit_buf[acc:acc + 1].copy_(verify_tokens[acc:acc + 1])
        if acc > 0:
            atlas.commit_kv_from_verify(gv, self.cache_len, acc)
            self.cache_len += acc
        return acc, [int(t) for t in draft_host[:acc]] + [int(verify_host[acc])]

    def exact_m1_verify(self, n_pend: int, draft_tokens: torch.Tensor) -> Tuple[int, int]:
        """Verify with the width-1 graph accelerated AR uses, stopping at the first mismatch
        (fast_generate.py:611-657).  Returns (accept_count, correction_or_bonus)."""
        bufs = self.bufs
        base = self.cache_len - n_pend
        g = None
        for j in range(n_pend):
            g = self.ar_step(bufs.pending_buf[j], base + j)
        pred = int(_argmax_rows(g.logits_out)[-1].item())
        acc = 0
        for j, token in enumerate(draft_tokens.tolist()):
            if int(token) != pred:
                break
            acc += 1
            g = self.ar_step(int(token), self.cache_len + j)
            pred = int(_argmax_rows(g.logits_out)[-1].item())
        self.cache_len += acc
        return acc, pred


def _empty_stats(prefill_time: float, seq_len: int, with_draft: bool) -> dict:
    """Statistics of a run that stopped on the first token (fast_generate.py:229-236,
    730-742)."""
    st = {"prefill_time": prefill_time, "decode_time": 1e-9, "total_time": prefill_time,
          "prefill_tokens": seq_len, "decode_tokens": 0, "timed_decode_tokens": 0,
          "untimed_output_tokens": 0, "n_iters": 0, "avg_accept": None, "ttft": prefill_time}
    if with_draft:
        st.update({"draft_iters": 0, "drafted_tokens": 0, "accepted_drafts": 0, "accept_rate": None,
                   "verifier_bonus_tokens": 0, "committed_tokens": 0, "committed_per_iter": None,
                   "conf_path_frac": None, "n_conf_path": 0, "n_verify_path": 0})
    return st


# --------------------------------------------------------------------------- AR
@torch.inference_mode()
def fast_ar_generate(model: Transformer, atlas: GraphAtlas, input_ids: torch.Tensor,
                     max_gen_len: int = 512, eos_ids=_BONSAI_EOS_IDS,
                     stop_strings: Optional[Sequence[str]] = None, tokenizer=None) -> Tuple[torch.Tensor, dict]:
    """Greedy AR decode with the captured width-1 graph (fast_generate.py:178-292): one
    replay and one host read per token.

    The next token stays on the device (the argmax writes it into the output buffer and the next
    replay's staging kernel gathers it from there), so the replay of token j + 1 is queued BEFORE the
    host reads token j: the read (an asynchronous copy to pinned memory plus an event) only decides
    when to stop.  A replay queued behind a token that turns out to be EOS, or to end a stop string,
    writes a staging row and an output slot past `gen_count`; neither is ever returned."""
    if 1 not in atlas.m_set:
        raise ValueError("atlas does not include M=1 for AR path")
    ses = _Session(model, atlas, input_ids, max_gen_len, eos_ids)
    bufs = ses.bufs
    prefill_time, next_tok, t0 = ses.start()
    if bufs.has_eos and next_tok in eos_ids:
        return bufs.gen_buf[:0].clone(), _empty_stats(prefill_time, ses.seq_len, with_draft=False)
    gen_count = 1                                  # tokens the host has seen
    launched = 1                                   # tokens whose replay has been queued (token 0: the prefill's)
    t1 = time.time()
    pipelined = bufs.gen_buf.is_cuda
    depth = 2 if pipelined else 1
    if pipelined:
        # the token's copy to the host runs on a stream of its own, behind an event, so that it does not sit
        # between two replays on the stream that computes
        host_tok = torch.empty(depth, dtype=torch.int64).pin_memory()
        seen = [torch.cuda.Event() for _ in range(depth)]
        made = [torch.cuda.Event() for _ in range(depth)]
        main, side = torch.cuda.current_stream(bufs.gen_buf.device), torch.cuda.Stream(bufs.gen_buf.device)
    last_dev = None
    top = atlas.segment_ladder[-1]
    while gen_count < max_gen_len:
        while (launched < max_gen_len and launched - gen_count < depth
               and (launched == 1 or ses.cache_len + 1 <= top)):
            ses.ensure_room()
            g = ses.ar_step(bufs.gen_buf[launched - 1:launched], ses.cache_len)
            ses.cache_len += 1
            slot = bufs.gen_buf[launched:launched + 1]
            last_dev = _argmax_rows(g.logits_out, bufs.argmax_out(slot))[-1:]
            if last_dev.data_ptr() != slot.data_ptr():
                slot.copy_(last_dev)
            if pipelined:
                k = launched % depth
                made[k].record(main)
                side.wait_event(made[k])
                with torch.cuda.stream(side):
                    host_tok[k:k + 1].copy_(slot, non_blocking=True)
                    seen[k].record(side)
            launched += 1
        if launched == gen_count:
            break                                  # the largest segment is full
        if pipelined:
            seen[gen_count % depth].synchronize()
            next_tok = int(host_tok[gen_count % depth])
        else:
            next_tok = int(last_dev.item())
        if bufs.has_eos and next_tok in eos_ids:
            break
        gen_count += 1
        if (stop_strings and tokenizer is not None
                and _decode_hits_stop(tokenizer, bufs.gen_buf[:gen_count].tolist(), stop_strings)):
            break
    torch.cuda.synchronize()
    decode_time = max(time.time() - t1, 1e-9)
    out = bufs.gen_buf[:gen_count].clone()
    n = int(out.numel())
    return out, {"prefill_time": prefill_time, "decode_time": decode_time,
                 "total_time": time.time() - t0, "prefill_tokens": ses.seq_len, "decode_tokens": n,
                 "timed_decode_tokens": max(0, n - 1), "untimed_output_tokens": min(1, n),
                 "n_iters": n, "avg_accept": 1.0, "ttft": prefill_time}


# --------------------------------------------------------------------------- draft/verify loops
def _draft_verify_generate(model, atlas, input_ids, *, policy: str, threshold: float,
                           hybrid_m: Optional[int], max_gen_len: int, eos_ids, use_fp8_draft: bool,
                           use_bf16_draft: bool, exact_m1_verify: bool) -> Tuple[torch.Tensor, dict]:
    """Engine of the speculative, hybrid and confidence policies.

    Every iteration replays one draft graph (materialising the pending rows and proposing
    D tokens).  Then, by policy:
      spec    always verify: commit draft[:acc] + the verifier's next token, n_pend := 1
      hybrid  if the confidence chain of this block reaches `hybrid_m`, commit the chain
              without verifying and carry it as pending (n_pend := chain); else verify
      conf    always commit the confidence chain
    (fast_generate.py:664-895 speculative, 902-1187 hybrid, 393-571 confidence)."""
    ses = _Session(model, atlas, input_ids, max_gen_len, eos_ids)
    bufs, D = ses.bufs, ses.D
    draft_role = _draft_role(atlas, use_fp8_draft, use_bf16_draft)
    verify_role = _verify_role(atlas) if policy != "conf" else None
    if hybrid_m is None:
        hybrid_m = 6 if D == 8 else (3 if D == 4 else max(1, (3 * D) // 4))

    prefill_time, next_tok, t0 = ses.start()
    # The confidence policy opens with a block of its own (fast_generate.py:322-351, 424-430): the last prompt
    # token re-fed as the anchor at its own position plus D - 1 mask rows, nothing pending, the history row of
    # the anchor hidden - a draft replay with n_pend = 0.  Its tokens are the request's untimed output and its
    # time belongs to the prefill, as in the reference.  The other policies take the prompt's greedy next token.
    first_block = policy == "conf"
    if first_block:
        bufs.pending_buf[0:1].copy_(ses.prompt_ids[-1:])
        n_pend, gen_count, n_iters = 0, 0, 0
    else:
        if bufs.has_eos and next_tok in eos_ids:
            return bufs.gen_buf[:0].clone(), _empty_stats(prefill_time, ses.seq_len, with_draft=True)
        bufs.pending_buf[0] = next_tok
        n_pend, gen_count, n_iters = 1, 1, 1
    untimed = gen_count
    eos_found = False
    n_conf_path = n_verify_path = draft_iters = drafted_total = 0
    accepted_draft_total = verifier_bonus_total = 0

    chain_out = bufs.chain_out(D)
    spec_draft_out = bufs.argmax_out(bufs.verify_rec[D + 2:2 * D + 2])
    t1 = time.time()
    while gen_count < max_gen_len and not eos_found:
        n_iters += 1
        draft_iters += 1
        drafted_total += D
        gd = ses.draft_step(n_pend, draft_role)

        draft_host = None                    # the D draft ids on the host, once read
        if policy == "spec":
            # the draft ids go beside the verifier's in the record that the host reads once
            draft_tokens = _argmax_rows(gd.logits_out, spec_draft_out)
            use_verify = True
            iter_accept = 0
            gv = None if exact_m1_verify else ses.stage_verify(n_pend, draft_tokens, verify_role)
        else:
            draft_tokens, iter_accept_t = _fused_draft_chain(gd.logits_out, threshold, chain_out)
            # The record's copy to the host is queued first, the verifier's inputs behind it, so that
            # their preparation overlaps the host's wait (fast_generate.py:1040-1055 queue them before a
            # blocking read).
            gv = None
            pending_read = _begin_read(bufs.chain_rec, draft_tokens, iter_accept_t)
            if policy == "hybrid" and not exact_m1_verify:
                gv = ses.stage_verify(n_pend, draft_tokens, verify_role)
            draft_host, n_host = _finish_read(pending_read)
            iter_accept = int(n_host[0])
            use_verify = policy == "hybrid" and iter_accept < hybrid_m

        commit_src = bufs.commit_buf          # device ids of this iteration's commit
        commit_host = None                    # the same ids on the host, when already read
        if not use_verify:
            commit_src = draft_tokens
            commit_host = [int(t) for t in draft_host[:iter_accept]]
            n_commit = accepted_this_iter = iter_accept
            bonus_this_iter = 0
            n_conf_path += 1
        else:
            if exact_m1_verify:
                acc, bonus = ses.exact_m1_verify(n_pend, draft_tokens)
                if acc > 0:
                    bufs.commit_buf[:acc].copy_(draft_tokens[:acc])
                bufs.commit_buf[acc] = bonus
            else:
                acc, commit_host = ses.verify_and_commit(gv, draft_tokens, draft_host)
            n_commit = acc + 1
            accepted_this_iter, bonus_this_iter = acc, 1
            n_verify_path += 1

        _, eos_hit, n_kept = _commit_and_eos(bufs, n_commit, eos_ids, commit_host)
        if eos_hit:
            eos_found = True
            n_commit = n_kept
        if gen_count + n_commit > max_gen_len:
            n_commit = max(0, max_gen_len - gen_count)

        # Attribute only what is emitted after EOS and length clipping: accepted drafts
        # first, the verifier's correction/bonus last (fast_generate.py:1106-1118).
        accepted_emitted = min(accepted_this_iter, n_commit)
        bonus_emitted = int(bool(bonus_this_iter) and n_commit > accepted_this_iter)
        if accepted_emitted + bonus_emitted != n_commit:
            raise RuntimeError(f"{policy} emitted-token accounting mismatch: accepted={accepted_emitted} "
                               f"bonus={bonus_emitted} committed={n_commit}")
        accepted_draft_total += accepted_emitted
        verifier_bonus_total += bonus_emitted

        if n_commit > 0:
            # ids -> output buffer; pending rows := the bonus token after a verified step (its rows were
            # promoted), or the whole committed block after a confidence commit (recomputed as pending next
            # time).  Written by the next draft replay's staging launch, or by the flush below.
            ses.defer_commit(commit_src, n_commit, use_verify, gen_count)
            gen_count += n_commit
        elif policy != "spec":
            eos_found = True
        if first_block:
            first_block = False
            untimed = gen_count
            torch.cuda.synchronize()
            prefill_time = time.time() - t0
            t1 = time.time()
        if eos_found or gen_count >= max_gen_len or n_commit <= 0:
            break
        n_pend = 1 if use_verify else n_commit
        if ses.out_of_room(n_pend):
            break

    ses.flush_commit()
    torch.cuda.synchronize()
    decode_time = max(time.time() - t1, 1e-9)
    out = bufs.gen_buf[:gen_count].clone()
    n_out = int(out.numel())
    if drafted_total != D * draft_iters:
        raise RuntimeError(f"{policy} drafted-token accounting mismatch")
    if draft_iters != n_conf_path + n_verify_path:
        raise RuntimeError(f"{policy} path/iteration accounting mismatch")
    prompt_token = 0 if policy == "conf" else 1             # outputs that came from the prompt's own logits
    if n_iters != draft_iters + prompt_token:
        raise RuntimeError(f"{policy} n_iters accounting mismatch")
    if n_out != prompt_token + accepted_draft_total + verifier_bonus_total:
        raise RuntimeError(f"{policy} output-origin accounting mismatch")
    if verifier_bonus_total > n_verify_path:
        raise RuntimeError(f"{policy} verifier bonus count exceeds verify paths")
    if accepted_draft_total > drafted_total:
        raise RuntimeError(f"{policy} accepted draft count exceeds drafted count")
    committed = n_out - prompt_token
    per_iter = committed / draft_iters if draft_iters > 0 else 0.0
    untimed = min(untimed, n_out)
    if policy == "conf" and n_out - untimed <= 0:
        decode_time = 1e-9                                  # everything came with the first block (fast_generate.py:436-441)
    return out, {
        "prefill_time": prefill_time, "decode_time": decode_time, "total_time": time.time() - t0,
        "prefill_tokens": ses.seq_len, "decode_tokens": n_out,
        "timed_decode_tokens": max(0, n_out - untimed), "untimed_output_tokens": untimed,
        "n_iters": n_iters, "avg_accept": per_iter, "ttft": prefill_time,
        "draft_iters": draft_iters, "drafted_tokens": drafted_total,
        "accepted_drafts": accepted_draft_total,
        "accept_rate": accepted_draft_total / drafted_total if drafted_total > 0 else 0.0,
        "verifier_bonus_tokens": verifier_bonus_total, "committed_tokens": committed,
        "committed_per_iter": per_iter,
        "conf_path_frac": n_conf_path / max(1, n_conf_path + n_verify_path),
        "n_conf_path": n_conf_path, "n_verify_path": n_verify_path,
    }


@torch.inference_mode()
def fast_speculative_generate(model: Transformer, atlas: GraphAtlas, input_ids: torch.Tensor,
                              max_gen_len: int = 512, eos_ids=_BONSAI_EOS_IDS,
                              use_fp8_draft: bool = False, use_fp8_verify: bool = False,
                              use_q1_verify: bool = False, use_w1a16_verify: bool = False,
                              exact_m1_verify: bool = False, rabv_margin: float = 0.0,
                              use_bf16_draft: bool = False) -> Tuple[torch.Tensor, dict]:
    """Self-speculative decode: draft D tokens, verify them with the width-(D+1) AR-causal
    graph (or the width-1 graph with `exact_m1_verify`), commit the matching prefix plus
    the verifier's own next token (fast_generate.py:664-895)."""
    validate_verification_options(rabv_margin, exact_m1_verify)
    validate_native_verifier(use_fp8_verify, use_q1_verify, use_w1a16_verify)
    return _draft_verify_generate(model, atlas, input_ids, policy="spec", threshold=0.0,
                                  hybrid_m=None, max_gen_len=max_gen_len, eos_ids=eos_ids,
                                  use_fp8_draft=use_fp8_draft, use_bf16_draft=use_bf16_draft,
                                  exact_m1_verify=exact_m1_verify)


@torch.inference_mode()
def fast_hybrid_generate(model: Transformer, atlas: GraphAtlas, input_ids: torch.Tensor,
                         threshold: float = 0.9, hybrid_m: Optional[int] = None,
                         max_gen_len: int = 512, eos_ids=_BONSAI_EOS_IDS, use_fp8_draft: bool = False,
                         use_bf16_draft: bool = False, use_fp8_verify: bool = False,
                         use_q1_verify: bool = False, use_w1a16_verify: bool = False,
                         exact_m1_verify: bool = False, rabv_margin: float = 0.0) -> Tuple[torch.Tensor, dict]:
    """Hybrid decode: a confidence chain of at least `hybrid_m` tokens is committed without
    verification, anything shorter falls back to the verifier (fast_generate.py:902-1187).
    Defaults: threshold 0.9, hybrid_m 6 for D=8 and 3 for D=4."""
    validate_verification_options(rabv_margin, exact_m1_verify)
    validate_native_verifier(use_fp8_verify, use_q1_verify, use_w1a16_verify)
    return _draft_verify_generate(model, atlas, input_ids, policy="hybrid", threshold=threshold,
                                  hybrid_m=hybrid_m, max_gen_len=max_gen_len, eos_ids=eos_ids,
                                  use_fp8_draft=use_fp8_draft, use_bf16_draft=use_bf16_draft,
                                  exact_m1_verify=exact_m1_verify)


@torch.inference_mode()
def fast_confidence_generate(model: Transformer, atlas: GraphAtlas, input_ids: torch.Tensor,
                             threshold: float = 0.9, max_gen_len: int = 512, eos_ids=_BONSAI_EOS_IDS,
                             use_fp8_draft: bool = False, use_bf16_draft: bool = False) -> Tuple[torch.Tensor, dict]:
    """Confidence-chain decode without verification (fast_generate.py:393-571).  The first block is
    the reference's ([last prompt token | MASK x (D-1)] over the prompt's K/V, nothing pending, its tokens
    the request's untimed output); the reference runs it as an eager variable-shape forward, here it is a
    replay of the width-D draft graph with n_pend = 0, like every later block."""
    return _draft_verify_generate(model, atlas, input_ids, policy="conf", threshold=threshold,
                                  hybrid_m=None, max_gen_len=max_gen_len, eos_ids=eos_ids,
                                  use_fp8_draft=use_fp8_draft, use_bf16_draft=use_bf16_draft,
                                  exact_m1_verify=False)
