"""Ring prefill attention for callers whose q / kv / o live in pinned HOST memory.

Attention heads are independent, so the job is cut into chunks of heads and pipelined over three streams: while the ring
pass of chunk c runs, the copy engines bring in chunk c+1 and take out the result of chunk c-1.  Only the first chunk's
upload and the last chunk's download are exposed.  The reference keeps these tensors on the device for the whole layer
(longserve_transformer_layer_infer.py:104-222); this is the host-buffer form of the same call, with the same buffer
layouts: q / o ``[tokens, Hq, D]``, kv ``[max_token_num, 2*Hkv, D]`` (K heads, then V heads).

A chunk of heads of such a tensor is a strided slab; it is moved with ``esp_memcpy_2d`` (one DMA descriptor per slab).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import _lib
from . import context_attention as ca
from . import ring as ringmod
from ._util import stream_ptr


def _copy2d(dst: int, dpitch: int, src: int, spitch: int, width: int, height: int, kind: int, stream: torch.cuda.Stream):
    _lib.check(_lib.attn().esp_memcpy_2d(dst, dpitch, src, spitch, width, height, kind, stream.cuda_stream), "esp_memcpy_2d")


class HostPrefillPipeline:
    """One instance's side of a ring prefill whose inputs and output are pinned host tensors.

    ``metas`` / ``stride`` / ``peers`` / ``comm`` / ``exchange`` as for ``ring.ring_context_attention`` (``comm`` may be None
    for a ring of one or when ``exchange`` carries the blocks).  With ``gather`` (a ``peer_ring.CopyEngineGather``) and
    ``lens`` (the requests' global lengths) every chunk runs as ``ring.gathered_context_attention`` instead: two launches per
    chunk, striped placement only.  ``head_chunks`` must divide the number of KV heads.  Device scratch: two chunk-sized
    sets of q / kv / o / m / l and, for an NCCL ring of more than one instance, two chunk-sized receive buffers."""

    def __init__(self, q_tokens: int, max_token_num: int, num_q_heads: int, num_kv_heads: int, head_dim: int, *, rank: int,
                 peers: Sequence[int], metas: Sequence["ringmod.BlockMeta"], stride: int, max_len_in_batch: int, comm=None,
                 head_chunks: int = 8, dtype=torch.bfloat16, device="cuda", overlap: bool = True, exchange=None,
                 gather=None, lens: Optional[Sequence[int]] = None):
        assert num_q_heads % num_kv_heads == 0 and num_kv_heads % head_chunks == 0
        self.Tq, self.Tkv, self.Hq, self.Hkv, self.D = q_tokens, max_token_num, num_q_heads, num_kv_heads, head_dim
        self.rank, self.peers, self.metas, self.stride, self.comm = rank, list(peers), metas, stride, comm
        self.max_len, self.overlap, self.exchange = max_len_in_batch, overlap, exchange
        self.gather, self.lens = gather, (list(lens) if lens is not None else None)
        if gather is not None:
            assert lens is not None and stride == len(self.peers) and self.peers == list(range(len(self.peers))), \
                "the gathered form needs the requests' lengths and a striped ring in rank order"
            self.plans = [ringmod.GatherPlan.build(self.lens, len(self.peers), r, device) for r in range(len(self.peers))]
        self.n = head_chunks
        self.kc = num_kv_heads // head_chunks                 # kv heads per chunk
        self.qc = self.kc * (num_q_heads // num_kv_heads)     # q heads per chunk
        self.dtype, self.device = dtype, torch.device(device)
        dev = self.device
        self.q = [torch.empty((q_tokens, self.qc, head_dim), dtype=dtype, device=dev) for _ in range(2)]
        self.kv = [torch.empty((max_token_num, 2 * self.kc, head_dim), dtype=dtype, device=dev) for _ in range(2)]
        self.o = [torch.empty((q_tokens, self.qc, head_dim), dtype=dtype, device=dev) for _ in range(2)]
        self.m = [torch.empty((q_tokens, self.qc), dtype=torch.float32, device=dev) for _ in range(2)]
        self.l = [torch.empty((q_tokens, self.qc), dtype=torch.float32, device=dev) for _ in range(2)]
        # with a copy-engine exchange the blocks arrive in the exchange's own buffers
        self.recv = ([torch.empty_like(self.kv[0]) for _ in range(2)]
                     if (len(self.peers) > 1 and exchange is None and gather is None) else [])
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self._ev = lambda: torch.cuda.Event()
        self._out_done: List[Optional[torch.cuda.Event]] = [None, None]     # o[b] has been copied out
        self._comp_done: List[Optional[torch.cuda.Event]] = [None, None]    # q[b] / kv[b] are no longer read

    def _upload(self, c: int, hq: torch.Tensor, hkv: torch.Tensor):
        b, es, D = c % 2, hq.element_size(), self.D
        s = self.s_in
        if self._comp_done[b] is not None:
            s.wait_event(self._comp_done[b])
        qw = self.qc * D * es
        _copy2d(self.q[b].data_ptr(), qw, hq.data_ptr() + c * qw, self.Hq * D * es, qw, self.Tq, 0, s)
        kw = self.kc * D * es
        src_pitch = 2 * self.Hkv * D * es
        _copy2d(self.kv[b].data_ptr(), 2 * kw, hkv.data_ptr() + c * kw, src_pitch, kw, self.Tkv, 0, s)                       # K heads
        _copy2d(self.kv[b].data_ptr() + kw, 2 * kw, hkv.data_ptr() + (self.Hkv * D * es) + c * kw, src_pitch, kw, self.Tkv, 0, s)  # V heads
        ev = self._ev(); ev.record(s)
        return ev

    def _init_state(self, o_, m_, l_):
        ca.init_attention_state(None, m_, l_)

    @torch.inference_mode()
    def run(self, hq: torch.Tensor, hkv: torch.Tensor, ho: torch.Tensor) -> torch.cuda.Event:
        """Enqueue the whole job; returns the event that completes when ``ho`` holds the result.  hq / ho
        ``[q_tokens, Hq, D]``, hkv ``[max_token_num, 2*Hkv, D]``: pinned, contiguous host tensors."""
        for t, shape in ((hq, (self.Tq, self.Hq, self.D)), (hkv, (self.Tkv, 2 * self.Hkv, self.D)), (ho, (self.Tq, self.Hq, self.D))):
            assert not t.is_cuda and t.is_pinned() and t.is_contiguous() and tuple(t.shape) == shape and t.dtype == self.dtype
        comp = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(comp)                 # everything queued before this call (e.g. the previous run) comes first
        self.s_out.wait_stream(comp)
        es, D = hq.element_size(), self.D
        in_ev = self._upload(0, hq, hkv)
        last = None
        for c in range(self.n):
            b = c % 2
            nxt = self._upload(c + 1, hq, hkv) if c + 1 < self.n else None
            comp.wait_event(in_ev)
            if self._out_done[b] is not None:
                comp.wait_event(self._out_done[b])
            q, kv, o, m, l = self.q[b], self.kv[b], self.o[b], self.m[b], self.l[b]
            me = self.metas[self.rank]
            if len(self.peers) == 1:
                self._init_state(o, m, l)
                ca.context_attention_fwd(q, kv[:, :self.kc], kv[:, self.kc:], o, me.start_loc, me.seq_len, me.first_idx, me.start_loc,
                                         me.seq_len, me.first_idx, self.stride, self.max_len, m, l)
            elif self.gather is not None:
                ringmod.gathered_context_attention(q, kv, o, m, l, rank=self.rank, lens=self.lens, P=len(self.peers),
                                                   metas=self.metas, plans=self.plans, max_len_in_batch=self.max_len,
                                                   num_kv_heads=self.kc, attention_fn=ca.context_attention_fwd,
                                                   init_fn=self._init_state, gather=self.gather)
            else:
                ringmod.ring_context_attention(q, kv, o, m, l, rank=self.rank, peers=self.peers, metas=self.metas, stride=self.stride,
                                               max_len_in_batch=self.max_len, num_kv_heads=self.kc, comm=self.comm,
                                               recv_buffers=self.recv, attention_fn=ca.context_attention_fwd,
                                               init_fn=self._init_state, overlap=self.overlap, exchange=self.exchange)
            done = self._ev(); done.record(comp)
            self._comp_done[b] = done
            self.s_out.wait_event(done)
            ow = self.qc * D * es
            _copy2d(ho.data_ptr() + c * ow, self.Hq * D * es, o.data_ptr(), ow, ow, self.Tq, 1, self.s_out)
            out = self._ev(); out.record(self.s_out)
            self._out_done[b] = out
            last = out
            in_ev = nxt
        comp.wait_event(last)                       # later work on the caller's stream sees the finished output
        return last
