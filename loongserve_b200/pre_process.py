"""Worker-side input preparation: turns the router's per-iteration description of a batch into the keyword
arguments of ``LlamaESPStack.forward`` — the job of ``prepare_prefill_inputs`` / ``prepare_decode_inputs`` in the
reference (loongserve/longserve_server/router/model_infer/pre_process.py:9-121 and :123-259), with the same names,
argument order, returned tuples and dictionary keys.

What differs from the reference, on purpose:

* all small integer vectors of one call are laid out in ONE pinned host buffer and reach the GPU in one asynchronous
  copy; sums and maxima are taken on the host lists, so no ``.item()`` round trip waits for the device
  (the reference builds one tensor per vector and reads ``sum`` / ``max`` back, pre_process.py:62,77,173,201);
* tensor parallelism inside an SP instance is out of scope: ``worker.tp_world_size`` must be 1, so the broadcasts
  of pre_process.py:59-75,169-172 have no counterpart;
* requests are looked up in ``batch.requests`` when the batch carries such a mapping, else in the module-level
  ``requests_mapping`` (the reference has only the global one, infer_batch.py).

A request record needs ``req_idx``, ``prompt_len``, ``cur_kv_len`` and ``running`` (the reference's
``req_status == RUNNING``).  As in the reference, ``prepare_decode_inputs`` increments ``prompt_len`` of the
requests this rank is the master of (pre_process.py:159).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

requests_mapping: Dict[object, "InferReq"] = {}


@dataclass
class InferReq:
    req_idx: int
    prompt_len: int
    cur_kv_len: int = 0
    running: bool = True


@dataclass
class InferBatch:
    request_ids: List[object]
    requests: Optional[Dict[object, InferReq]] = None

    def __len__(self):
        return len(self.request_ids)


@dataclass
class Worker:
    """The three attributes of the reference's worker that input preparation reads, plus the target device."""
    sp_rank: int = 0
    tp_rank: int = 0
    tp_world_size: int = 1
    device: object = "cuda"


class _Packer:
    """Collects int32 vectors, then uploads them as one buffer; each vector starts on a 16-byte boundary."""

    def __init__(self):
        self._chunks: List[np.ndarray] = []
        self._spans = []
        self._n = 0

    def add(self, values: Sequence[int]) -> int:
        a = np.asarray(values, dtype=np.int32).reshape(-1)
        self._chunks.append(a)
        self._spans.append((self._n, a.size))
        self._n += (a.size + 3) // 4 * 4
        return len(self._spans) - 1

    def upload(self, device) -> List[torch.Tensor]:
        host = torch.zeros(max(self._n, 4), dtype=torch.int32, pin_memory=torch.cuda.is_available())
        hv = host.numpy()
        for a, (off, n) in zip(self._chunks, self._spans):
            hv[off:off + n] = a
        dev = host.to(device, non_blocking=True)
        return [dev[off:off + n] for off, n in self._spans]


def _lookup(batch):
    reqs = getattr(batch, "requests", None)
    return reqs if reqs is not None else requests_mapping


def _check_worker(worker):
    if worker.tp_world_size != 1 or worker.tp_rank != 0:
        raise NotImplementedError("tensor parallelism inside an SP instance is out of scope (tp_world_size must be 1)")


def prepare_prefill_inputs(batch, global_input_kvargs: tuple, worker):
    """``global_input_kvargs`` = (input_ids, max_token_num, occupied_instances, logical_sp_rank, should_decode,
    need_context_migration, kv_cache_index_begin, kv_cache_index_end) as the router sends it to a driver worker
    (pre_process.py:15); ``input_ids[i]`` are the token ids of request i that live on this instance.
    Returns ``(kwargs, run_reqs, not_run_reqs)``; ``kwargs`` is empty when nothing runs."""
    _check_worker(worker)
    (input_ids, max_token_num, occupied_instances, logical_sp_rank, _should_decode, need_context_migration,
     cache_begin, cache_end) = global_input_kvargs
    reqs = _lookup(batch)
    logical_sp_peer_ranks = [sp_i * worker.tp_world_size + worker.tp_rank for sp_i in occupied_instances]

    run_reqs, not_run_reqs = [], []
    req_idx, start_loc, seq_len, ids = [], [], [], []
    total = 0
    for i, request_id in enumerate(batch.request_ids):
        req = reqs[request_id]
        assert req.running
        if req.cur_kv_len != 0:                      # already prefilled: not part of this call
            not_run_reqs.append(req)
            continue
        run_reqs.append(req)
        req_idx.append(req.req_idx)
        start_loc.append(total)
        n = len(input_ids[i])
        if n > 0:
            ids.append(np.asarray(input_ids[i], dtype=np.int64))
        seq_len.append(n)
        total += n
    if not run_reqs:
        return {}, run_reqs, not_run_reqs

    bs = len(run_reqs)
    device = getattr(worker, "device", "cuda")
    pk = _Packer()
    pk.add(req_idx); pk.add(start_loc); pk.add(seq_len); pk.add([logical_sp_rank] * bs)
    if need_context_migration:
        # one entry per request that runs, in the same order (the router builds them that way, manager.py:764-803)
        assert len(cache_begin) == bs and len(cache_end) == bs
        pk.add(cache_begin); pk.add(cache_end)
    vec = pk.upload(device)
    ids_host = torch.from_numpy(np.concatenate(ids) if ids else np.zeros(0, dtype=np.int64))
    if torch.cuda.is_available():
        ids_host = ids_host.pin_memory()
    kwargs = {
        "batch_size": bs,
        "total_token_num": total,
        "max_token_num": max_token_num,
        "max_len_in_batch": max(seq_len),
        "input_ids": ids_host.to(device, non_blocking=True),
        "b_req_idx": vec[0],
        "b_start_loc": vec[1],
        "b_seq_len": vec[2],
        "first_token_global_idx": vec[3],
        "sp_master_rank": None,
        "logical_sp_peer_ranks": logical_sp_peer_ranks,
        "logical_sp_rank": logical_sp_rank,
        "newkv_alloc_sp_rank": None,
        "peer_sp_master_rank_list": None,
        "peer_query_buffer_range_list": None,
        "peer_batch_size": None,
        "peer_max_len_in_batch": None,
        "peer_b_req_idx": None,
        "peer_b_seq_len": None,
        "need_context_migration": need_context_migration,
        "kv_cache_index_begin": vec[4] if need_context_migration else None,
        "kv_cache_index_end": vec[5] if need_context_migration else None,
        "multimodal_params": None,
        "is_prefill": True,
    }
    return kwargs, run_reqs, not_run_reqs


def prepare_decode_inputs(batch, global_input_kvargs: tuple, worker):
    """``global_input_kvargs`` = (input_ids, first_token_global_idx, num_sp_master_ranks, mini_batch_size_list,
    occupied_instances, logical_sp_rank) (pre_process.py:129).  The first ``num_sp_master_ranks`` logical ranks are
    masters; master k owns the k-th slice of ``batch.request_ids`` (sizes in ``mini_batch_size_list``) and every
    rank serves, as a peer, all requests it is not the master of, in batch order.
    Returns ``(kwargs, run_reqs, peer_run_reqs, not_run_reqs)``."""
    _check_worker(worker)
    input_ids, first_token_global_idx, num_masters, mini_sizes, occupied_instances, logical_sp_rank = global_input_kvargs
    reqs = _lookup(batch)
    logical_sp_peer_ranks = [sp_i * worker.tp_world_size + worker.tp_rank for sp_i in occupied_instances]
    device = getattr(worker, "device", "cuda")

    bounds = np.concatenate([[0], np.cumsum(np.asarray(mini_sizes, dtype=np.int64))]).tolist()
    ranges = [(int(bounds[k]), int(bounds[k + 1])) for k in range(len(mini_sizes))]
    is_master = logical_sp_rank < num_masters
    n_req = len(batch.request_ids)
    lo, hi = ranges[logical_sp_rank] if is_master else (n_req, n_req)
    mine = batch.request_ids[lo:hi] if is_master else None
    others = batch.request_ids[:lo] + batch.request_ids[hi:] if is_master else batch.request_ids

    run_reqs, peer_run_reqs, not_run_reqs = [], [], []
    pk = _Packer()
    slots = {}
    bs, total, max_len, ids_dev = 0, None, 0, None
    if mine is not None:
        bs = total = len(mine)
        idx, lens = [], []
        for request_id in mine:
            req = reqs[request_id]
            assert req.running
            run_reqs.append(req)
            idx.append(req.req_idx)
            req.prompt_len += 1                      # the length seen by the kernels includes the new token
            assert req.cur_kv_len == req.prompt_len - 1, f"{request_id}: {req.cur_kv_len} != {req.prompt_len - 1}"
            lens.append(req.prompt_len)
        slots["b_req_idx"] = pk.add(idx)
        slots["b_seq_len"] = pk.add(lens)
        slots["first"] = pk.add(first_token_global_idx)
        max_len = max(lens) if lens else 0
        ids_host = torch.from_numpy(np.asarray(input_ids, dtype=np.int64).reshape(-1))
        if torch.cuda.is_available():
            ids_host = ids_host.pin_memory()
        ids_dev = ids_host.to(device, non_blocking=True)
    peer_bs, peer_max = None, 0
    if others:
        idx, lens = [], []
        for request_id in others:
            req = reqs[request_id]
            assert req.running
            peer_run_reqs.append(req)
            idx.append(req.req_idx)
            assert req.cur_kv_len == req.prompt_len, f"{req.cur_kv_len} != {req.prompt_len}"
            lens.append(req.prompt_len)
        peer_bs, peer_max = len(others), max(lens)
        slots["peer_b_req_idx"] = pk.add(idx)
        slots["peer_b_seq_len"] = pk.add(lens)
    assert len(run_reqs) + len(peer_run_reqs) == n_req
    if n_req == 0:
        return {}, run_reqs, peer_run_reqs, not_run_reqs
    vec = pk.upload(device)

    def v(name):
        return vec[slots[name]] if name in slots else None

    own = hi - lo
    peer_masters = [sp_i for k, sp_i in enumerate(logical_sp_peer_ranks[:num_masters]) if k != logical_sp_rank]
    # the peer query buffer holds the other masters' mini-batches back to back: positions after this rank's own
    # slice shift down by its size
    peer_ranges = [(ranges[k][0] - (own if k > logical_sp_rank else 0), ranges[k][1] - (own if k > logical_sp_rank else 0))
                   for k in range(num_masters) if k != logical_sp_rank]
    kwargs = {
        "batch_size": bs,
        "total_token_num": total,
        "max_token_num": None,
        "max_len_in_batch": max_len,
        "input_ids": ids_dev,
        "b_req_idx": v("b_req_idx"),
        "b_start_loc": None,
        "b_seq_len": v("b_seq_len"),
        "first_token_global_idx": v("first"),
        "sp_master_rank": logical_sp_peer_ranks[logical_sp_rank] if is_master else None,
        "logical_sp_peer_ranks": logical_sp_peer_ranks,
        "logical_sp_rank": logical_sp_rank,
        "newkv_alloc_sp_rank": None,
        "peer_sp_master_rank_list": peer_masters or None,
        "peer_query_buffer_range_list": peer_ranges,
        "peer_batch_size": peer_bs,
        "peer_max_len_in_batch": peer_max,
        "peer_b_req_idx": v("peer_b_req_idx"),
        "peer_b_seq_len": v("peer_b_seq_len"),
        "need_context_migration": False,
        "kv_cache_index_begin": None,
        "kv_cache_index_end": None,
        "multimodal_params": None,
        "is_prefill": False,
    }
    return kwargs, run_reqs, peer_run_reqs, not_run_reqs
