"""A Llama-architecture layer stack around the ESP attention runtime: what the reference's pre / transformer /
post layer-infer classes do for one SP instance with tp = 1
(loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:70-96, 372-456;
longserve_pre_layer_infer.py:35-43; longserve_post_layer_infer.py:37-83), with random-initialised weights in the
reference's fused layouts (layer_weights/longserve_transformer_layer_weight.py:60-117):
``q_weight_ [hidden, Hq*D]``, ``kv_weight_ [hidden, 2*Hkv*D]``, ``o_weight_ [Hq*D, hidden]``,
``gate_up_proj [hidden, 2*F]``, ``down_proj [F, hidden]``.

Projections are cuBLAS (``torch.mm``), exactly as in the reference; everything else runs in this package's kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import layer_ops
from .attention_runtime import ESPAttentionRuntime


@dataclass
class LlamaConfig:
    num_layers: int = 32
    hidden: int = 4096
    num_q_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    rms_eps: float = 1e-5
    rope_base: float = 10000.0


class LlamaWeights:
    """Seeded random weights (normal, std 0.02; norm weights 1 + small noise)."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device="cuda", seed: int = 0):
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)

        def nw(n):
            return (1.0 + 0.1 * torch.randn(n, generator=g, device=device, dtype=torch.float32)).to(dtype)

        H, Hq, Hkv, D, F = cfg.hidden, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim, cfg.ffn
        self.embed = w(cfg.vocab, H)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(att_norm=nw(H), q=w(H, Hq * D), kv=w(H, 2 * Hkv * D), o=w(Hq * D, H), ffn_norm=nw(H),
                                    gate_up=w(H, 2 * F), down=w(F, H)))
        self.final_norm = nw(H)
        self.lm_head = w(H, cfg.vocab)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, base: float, dtype):
    """cos/sin rows for the given global positions (rotate-half convention), built in fp32 then cast, as the
    reference's table is (longserve_model.py:264-275)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = torch.outer(positions.to(torch.float32), inv_freq)
    return torch.cos(ang).to(dtype).contiguous(), torch.sin(ang).to(dtype).contiguous()


class LlamaESPStack:
    def __init__(self, cfg: LlamaConfig, weights: LlamaWeights, runtime: ESPAttentionRuntime):
        self.cfg, self.w, self.rt = cfg, weights, runtime

    # ------------------------------------------------------------------ prefill (every instance of the ring)
    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor, positions: torch.Tensor, st, last_token_rows: Optional[torch.Tensor] = None):
        """input_ids / positions: this instance's local tokens (packed, request-major) and their global positions;
        ``st`` from ``ESPAttentionRuntime.prepare_prefill``.  Returns logits of ``last_token_rows`` (local row
        indices; default: none -> hidden states are returned instead)."""
        cfg, rt = self.cfg, self.rt
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        x = self.w.embed[input_ids.long()]
        n = x.shape[0]
        cos, sin = rope_cos_sin(positions, D, cfg.rope_base, x.dtype)
        for li, lw in enumerate(self.w.layers):
            h = layer_ops.rms_norm(x, lw["att_norm"], cfg.rms_eps)
            q = torch.mm(h, lw["q"])
            cache_kv = rt.pre_cache_kv(st, li)
            torch.mm(h, lw["kv"], out=cache_kv.view(-1, 2 * Hkv * D)[:n])
            layer_ops.rotary_emb(q.view(-1, Hq, D), cache_kv[:n, :Hkv, :], cos, sin)
            o = rt.context_attention(q.view(-1, Hq, D), st, li, out=h.view(-1, Hq, D) if Hq * D == cfg.hidden else None)
            x.add_(torch.mm(o.view(n, Hq * D), lw["o"]))
            x.add_(layer_ops.ffn_block(x, lw["ffn_norm"], cfg.rms_eps, lw["gate_up"], lw["down"]))
        if last_token_rows is None:
            return x
        return self._logits(x[last_token_rows.long()])

    # ------------------------------------------------------------------ decode
    @torch.inference_mode()
    def decode(self, input_ids: Optional[torch.Tensor], positions: Optional[torch.Tensor], st):
        """One decode step.  Masters pass their requests' new token ids and global positions and get logits;
        pure peers pass None and only serve attention for the other masters' queries."""
        cfg, rt = self.cfg, self.rt
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        is_master = st.master_plan is not None
        if is_master:
            x = self.w.embed[input_ids.long()]
            n = x.shape[0]
            cos, sin = rope_cos_sin(positions, D, cfg.rope_base, x.dtype)
        for li, lw in enumerate(self.w.layers):
            if is_master:
                h = layer_ops.rms_norm(x, lw["att_norm"], cfg.rms_eps)
                q = torch.mm(h, lw["q"])
                cache_kv = rt.decode_cache_kv(st, li)
                torch.mm(h, lw["kv"], out=cache_kv.view(-1, 2 * Hkv * D)[:n])
                layer_ops.rotary_emb(q.view(-1, Hq, D), cache_kv[:n, :Hkv, :], cos, sin)
                rt.post_decode_cache_kv(st, li)
                o = rt.token_attention(q.view(-1, Hq, D), st, li)
                x.add_(torch.mm(o.view(n, Hq * D), lw["o"]))
                x.add_(layer_ops.ffn_block(x, lw["ffn_norm"], cfg.rms_eps, lw["gate_up"], lw["down"]))
            else:
                rt.token_attention(None, st, li)
        return self._logits(x) if is_master else None

    # ------------------------------------------------------------------ the reference's call surface
    @torch.inference_mode()
    def forward(self, batch_size, total_token_num, max_token_num, max_len_in_batch, input_ids, b_req_idx, b_start_loc,
                b_seq_len, first_token_global_idx, sp_master_rank, logical_sp_peer_ranks, logical_sp_rank,
                newkv_alloc_sp_rank=None, peer_sp_master_rank_list=None, peer_query_buffer_range_list=None,
                peer_batch_size=None, peer_max_len_in_batch=None, peer_b_req_idx=None, peer_b_seq_len=None,
                need_context_migration=False, kv_cache_index_begin=None, kv_cache_index_end=None, multimodal_params=None,
                is_prefill=True):
        """Same keyword arguments as ``LongServeLlamaModel.forward`` (loongserve/models/llama/longserve_model.py:279-321),
        as built by the worker's ``prepare_prefill_inputs`` / ``prepare_decode_inputs``.  Prefill returns the logits of
        every request's last local token (longserve_post_layer_infer.py:37-43), decode the logits on the master."""
        rt = self.rt
        P = len(logical_sp_peer_ranks)
        if is_prefill:
            st = rt.prepare_prefill(batch_size, total_token_num, max_token_num, max_len_in_batch, b_req_idx, b_start_loc, b_seq_len,
                                    first_token_global_idx, logical_sp_peer_ranks, logical_sp_rank, need_context_migration,
                                    kv_cache_index_begin, kv_cache_index_end, striped=True)
            # global position of local row i of a request = first + i * P (longserve_infer_struct.py:112-126)
            lens64 = b_seq_len.long()
            req_of_tok = torch.repeat_interleave(torch.arange(batch_size, device=lens64.device), lens64)
            local = torch.arange(total_token_num, device=lens64.device) - b_start_loc.long()[req_of_tok]
            positions = first_token_global_idx.long()[req_of_tok] + local * P
            last_rows = (b_start_loc.long() + lens64 - 1).clamp_min(0)
            return self.prefill(input_ids, positions, st, last_token_rows=last_rows)
        is_master = sp_master_rank == rt.total_rank_
        st = rt.prepare_decode(batch_size, total_token_num, max_len_in_batch, b_req_idx, b_seq_len, first_token_global_idx,
                               sp_master_rank, logical_sp_peer_ranks, logical_sp_rank, peer_sp_master_rank_list,
                               peer_query_buffer_range_list, peer_batch_size or 0, peer_max_len_in_batch or 0, peer_b_req_idx,
                               peer_b_seq_len)
        return self.decode(input_ids if is_master else None, first_token_global_idx if is_master else None, st)

    def _logits(self, x):
        h = layer_ops.rms_norm(x.contiguous(), self.w.final_norm, self.cfg.rms_eps)
        return torch.mm(h, self.w.lm_head).float()


class GraphedDecode:
    """One decode iteration of an ESP group (all layers, the attention exchange over peer memory, logits) recorded
    once per instance into a CUDA graph and replayed every step, so that a step costs one graph launch instead of
    a few hundred kernel launches issued from Python.  The reference issues every kernel of every layer from Python
    (longserve_transformer_layer_infer.py:372-456) and allocates its per-step buffers anew (longserve_model.py:438-538).

    Everything that changes from step to step lives in fixed device buffers the graph reads: the new token ids, the
    pool slots of the new tokens, the requests' local lengths and positions (advanced inside the graph), and the base
    of the exchange's flag values (``FusedDecodeGroup.step(step_value=, value_base=)``), advanced by one per layer
    inside the graph.  Grid sizes are recorded for ``max_new_tokens`` more tokens than the longest request has now;
    sequence blocks beyond a request's current length return at once.

    Single master per group (instance ``group.master``); every instance of the group builds one of these, calls
    ``capture()`` once and then ``step()`` the same number of times.
    """

    def __init__(self, stack: LlamaESPStack, group, b_req_idx: torch.Tensor, b_seq_len: torch.Tensor,
                 positions: Optional[torch.Tensor] = None, max_new_tokens: int = 128, block_seq: Optional[int] = None):
        """``b_req_idx`` / ``b_seq_len``: the master's requests as stored on THIS instance (int32; on the master the
        lengths exclude the token the first step adds).  ``positions`` (master only): global position of the first new
        token of every request."""
        self.stack, self.group = stack, group
        rt, cfg = stack.rt, stack.cfg
        self.is_master = group.rank == group.master
        dev = b_seq_len.device
        B = b_seq_len.shape[0]
        self.B = B
        longest = int(b_seq_len.max())                                   # set-up time read-back
        self.bound = longest + (int(max_new_tokens) if self.is_master else 0)
        self.block_seq = int(block_seq or rt.decode_block_seq or 256)
        nblk = (self.bound + self.block_seq - 1) // self.block_seq
        f32 = dict(dtype=torch.float32, device=dev)
        Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
        self.b_req_idx = b_req_idx.to(torch.int32).contiguous().clone()
        self.seq_len = b_seq_len.to(torch.int32).contiguous().clone()
        self.mid_o = torch.empty((nblk, B, Hq, D), **f32)
        self.mid_lse = torch.empty((nblk, B, Hq), **f32)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self._synced = None
        if self.is_master:
            assert positions is not None and positions.shape[0] == B
            self.pos = positions.to(torch.int64).contiguous().clone()
            self.input_ids = torch.zeros(B, dtype=torch.int64, device=dev)
            self.new_slots = torch.zeros(B, dtype=torch.int64, device=dev)
            self.kv_scratch = torch.empty((B, 2 * Hkv, D), dtype=rt.dtype, device=dev)
            self.out_lse = torch.empty((B, Hq), **f32)
            self.logits = torch.empty((B, cfg.vocab), **f32)
        self.graph = None
        self.steps_left = int(max_new_tokens)

    @torch.inference_mode()
    def _record(self):
        stack, rt, cfg, grp = self.stack, self.stack.rt, self.stack.cfg, self.group
        Hq, Hkv, D, B = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim, self.B
        rtt = rt.req_manager.req_to_token_indexs
        L = cfg.num_layers
        if not self.is_master:
            for li in range(L):
                grp.step(None, rt.mem_manager.kv_buffer[li], rtt, Hkv, self.b_req_idx, self.seq_len, self.bound, self.block_seq,
                         self.mid_o, self.mid_lse, step_value=li + 1, value_base=self.counter)
            self.counter.add_(L)
            return
        from . import kv_ops
        self.seq_len.add_(1)                                             # lengths now include the new token
        kv_ops.copy_kv_index_to_req(rtt, self.b_req_idx, self.seq_len, self.new_slots)
        x = stack.w.embed[self.input_ids]
        cos, sin = rope_cos_sin(self.pos, D, cfg.rope_base, x.dtype)
        for li, lw in enumerate(stack.w.layers):
            pool = rt.mem_manager.kv_buffer[li]
            h = layer_ops.rms_norm(x, lw["att_norm"], cfg.rms_eps)
            q = torch.mm(h, lw["q"])
            torch.mm(h, lw["kv"], out=self.kv_scratch.view(B, 2 * Hkv * D))
            layer_ops.rotary_emb(q.view(B, Hq, D), self.kv_scratch[:, :Hkv, :], cos, sin)
            kv_ops.destindex_copy_kv(self.kv_scratch, self.new_slots, pool)
            o, _ = grp.step(q.view(B, Hq, D), pool, rtt, Hkv, self.b_req_idx, self.seq_len, self.bound, self.block_seq,
                            self.mid_o, self.mid_lse, out_lse=self.out_lse, step_value=li + 1, value_base=self.counter)
            x.add_(torch.mm(o.view(B, Hq * D), lw["o"]))
            x.add_(layer_ops.ffn_block(x, lw["ffn_norm"], cfg.rms_eps, lw["gate_up"], lw["down"]))
        self.logits.copy_(stack._logits(x))
        self.pos.add_(1)
        self.counter.add_(L)

    def capture(self):
        """Record the step.  Nothing runs on the GPU here; run at least one ordinary decode step on this process
        first so that library workspaces exist."""
        grp = self.group
        if self.is_master and (grp._ones is None or grp._ones.shape[0] != self.B):
            # the merge over the P partial slots reads this constant; it must hold its value before the first replay
            grp._ones = torch.full((self.B,), grp.world, dtype=torch.int32, device=self.seq_len.device)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._record()
        return self

    @torch.inference_mode()
    def step(self, input_ids: Optional[torch.Tensor] = None, new_slots: Optional[torch.Tensor] = None):
        """Replay one step.  Master: ``input_ids`` [B] (device or host) are the tokens to feed, ``new_slots`` [B] the
        pool slots their K/V rows go to (default: allocated from the runtime's pool manager); returns the logits
        buffer [B, vocab] (overwritten by the next step).  Peers pass nothing and get None."""
        assert self.graph is not None, "call capture() first"
        assert self.steps_left > 0, "the graph was recorded for max_new_tokens steps"
        grp, L = self.group, self.stack.cfg.num_layers
        if self._synced != grp.step_id:                                  # steps ran outside the graph since the last replay
            self.counter.fill_(grp.step_id)
        if self.is_master:
            if new_slots is None:
                new_slots = self.stack.rt.mem_manager.alloc(self.B)
            self.new_slots.copy_(new_slots, non_blocking=True)
            self.input_ids.copy_(input_ids, non_blocking=True)
        self.graph.replay()
        grp.advance(L)
        self._synced = grp.step_id
        self.steps_left -= 1
        return self.logits if self.is_master else None
