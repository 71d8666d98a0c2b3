"""Test scaffolding: a GraphAtlas whose graphs replay the CPU oracle forward.

Lets the package's own decode loops (bitmtp_b200.fast_generate) run without a GPU, so the
host logic (input rows, width selection, segment migration, KV promotion, accounting) can
be checked against the token streams recorded from the reference's loops.  Only tests
import this module.
"""
import types

import numpy as np
import torch

from bitmtp_b200 import fast_generate as FG
from bitmtp_b200.fast_runtime import GraphAtlas, role_logit_rows
from oracle import oracle as O

PREFILL_CHUNK = 16


class OracleModel:
    """`.args` + the chunked integer prefill, backed by oracle.OracleModel."""

    def __init__(self, om, args):
        self.om, self.args = om, args

    def forward_sdlm_prefill(self, token_values, cache, positions=None, block_size=1, fast=False,
                             causal_attn=True):
        om = self.om
        seq = int(token_values.shape[0])
        kv = om.new_kv(seq, PREFILL_CHUNK)
        logits = np.empty((seq, om.vocab), dtype=np.float32)
        toks = token_values.numpy()
        for c0 in range(0, seq, PREFILL_CHUNK):
            n = min(PREFILL_CHUNK, seq - c0)
            logits[c0:c0 + n] = om.forward(toks[c0:c0 + n], np.arange(c0, c0 + n), kv, sigma=c0,
                                           role=O.ROLE_AR, cache_len=c0, n_pend=0)
        for i in range(om.L):
            cache[i] = (O.u16_to_torch(kv[0, i, :, :, :seq, :].copy()),
                        O.u16_to_torch(kv[1, i, :, :, :seq, :].copy()))
        return torch.from_numpy(logits)


class CpuAtlas(GraphAtlas):
    """GraphAtlas with the capture replaced by oracle-backed replay objects; selection,
    commit and migration logic is the package's own, with the row copies done by torch."""

    def __init__(self, om, args, segment_ladder, m_set, roles):
        self.model, self.args = None, args
        self.device, self.dtype = torch.device("cpu"), torch.bfloat16
        self.segment_ladder = tuple(sorted(set(segment_ladder)))
        self.m_set = tuple(sorted(set(m_set)))
        self.roles = tuple(roles)
        self.D, self.M_max = args.block_size, max(m_set)
        self.vocab_size, self.n_layers = args.vocab_size, args.n_layers
        self.n_kv, self.head_dim = args.n_kv_heads, args.head_dim
        self.kv_buffers = {s: torch.zeros(2, self.n_layers, 1, self.n_kv, s + self.M_max, 128,
                                          dtype=torch.bfloat16) for s in self.segment_ladder}
        self._allocate_input_bufs()
        self.graphs = {}
        self.log = []
        for sigma in self.segment_ladder:
            kv_np = self.kv_buffers[sigma].view(torch.int16).numpy().view(np.uint16)
            for M in self.m_set:
                for role in (("ar",) if M == 1 else tuple(r for r in roles if r != "ar")):
                    if M == 1 and "ar" not in roles:
                        continue
                    ls, le = role_logit_rows(role, M, self.D)
                    g = types.SimpleNamespace(
                        tokens_buf=self.tokens_m[M], positions_buf=self.positions_m[M], attn_mask=None,
                        logits_out=torch.zeros(le - ls, args.vocab_size), M=M, sigma=sigma, role=role,
                        P=M - self.D, logits_start=ls, logits_end=le, state=None)

                    def replay(g=g, kv_np=kv_np):
                        cache_len, n_pend = g.state
                        self.log.append((g.role, g.M, g.sigma, cache_len, n_pend))
                        lg = om.forward(g.tokens_buf.numpy(), g.positions_buf.numpy(), kv_np, g.sigma,
                                        O.ROLE_IDS[g.role], cache_len, n_pend, g.logits_start,
                                        g.logits_end)
                        g.logits_out.copy_(torch.from_numpy(lg))

                    g.cuda_graph = types.SimpleNamespace(replay=replay)
                    self.graphs[(M, sigma, role)] = g

    def prepare_step(self, graph, cache_len, n_pend, causal_attn=True):
        if graph.role == "verify" and cache_len <= 0:
            raise RuntimeError("batched verifier requires a committed anchor")
        graph.state = (int(cache_len), max(0, min(int(n_pend), max(graph.P, 0))))

    def _copy_rows(self, sigma, src, dst, n):
        buf = self.kv_buffers[sigma]
        buf[:, :, :, :, dst:dst + n, :] = buf[:, :, :, :, src:src + n, :].clone()

    def commit_kv(self, graph, cache_len, n_accept):
        if n_accept > 0:
            self._copy_rows(graph.sigma, graph.sigma, cache_len, n_accept)

    def commit_kv_from_verify(self, verify_graph, cache_len, n_accept):
        if n_accept > 0:
            self._copy_rows(verify_graph.sigma, verify_graph.sigma + 1, cache_len, n_accept)


class patched_host_ops:
    """Context manager: route the loops' three device reductions to the oracle and make
    torch.cuda.synchronize a no-op; `policy` (synthetic.AcceptancePolicy) may replace the
    measured counts."""

    def __init__(self, D, policy):
        self.D, self.policy = D, policy

    def __enter__(self):
        self.saved = (FG._argmax_rows, FG._fused_draft_chain, FG._fused_verify_accept,
                      torch.cuda.synchronize)
        policy = self.policy

        # The loops offer result buffers (`out`); these stand-ins return fresh tensors instead, which
        # takes the loops through their one-read-per-part path.
        def argmax_rows(logits, out=None):
            return torch.from_numpy(O.argmax_rows(logits.numpy()))

        def chain(logits, threshold, out=None):
            idx, n, _ = O.draft_chain(logits.numpy(), float(threshold))
            a = policy.chain_count()
            return torch.from_numpy(idx), torch.tensor([n if a is None else a])

        def accept(draft, verify, Dd, out=None):
            a = policy.accept_count()
            return torch.tensor([O.verify_accept(draft.numpy(), verify.numpy(), Dd) if a is None else a])

        FG._argmax_rows, FG._fused_draft_chain, FG._fused_verify_accept = argmax_rows, chain, accept
        torch.cuda.synchronize = lambda *a, **k: None
        return self

    def __exit__(self, *exc):
        (FG._argmax_rows, FG._fused_draft_chain, FG._fused_verify_accept,
         torch.cuda.synchronize) = self.saved
        return False
