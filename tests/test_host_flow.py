"""Host-side flow around the path, on CPU: the scheduling search picks the batch and its instances, the worker-side
preparation builds every instance's keyword arguments, and a ring over exactly those arguments (oracle ring steps)
reproduces single-device causal attention.  Ties router/manager.py:687-760, pre_process.py:9-121 and
longserve_transformer_layer_infer.py:104-178 together the way a prefill iteration uses them."""
import numpy as np
import torch

from loongserve_b200 import pre_process as pp
from loongserve_b200 import scheduler
from oracle import esp_oracle as O


def test_schedule_prepare_and_ring_agree_with_full_attention():
    rng = np.random.RandomState(2)
    lens = sorted((int(x) for x in rng.randint(40, 400, size=5)), reverse=True)           # longest first, as the router sorts
    n_inst = 4
    left = [2000] * n_inst
    abc = np.vstack([[np.nan] * 3] + [[0.02 + 0.004 * u, 4e-5 / u, 2.5e-10 / u] for u in range(1, n_inst + 1)])
    batches, cost, longest = scheduler.plan_prefill_batches(lens, left, abc)
    assert sum(b[0].stop - b[0].start for b in batches) == len(lens) and np.isfinite(cost) and longest > 0
    g = torch.Generator().manual_seed(0)
    Hq, Hkv, D = 2, 1, 32
    for req_slice, inst_slice in batches:
        blens = lens[req_slice]
        instances = list(range(n_inst))[inst_slice]
        P = len(instances)
        T = sum(blens)
        ids = torch.randint(0, 1000, (T,), generator=g)
        q = torch.randn(T, Hq, D, generator=g); k = torch.randn(T, Hkv, D, generator=g); v = torch.randn(T, Hkv, D, generator=g)
        starts = np.concatenate([[0], np.cumsum(blens)[:-1]])
        reqs = {f"r{i}": pp.InferReq(req_idx=i, prompt_len=n, cur_kv_len=0) for i, n in enumerate(blens)}
        batch = pp.InferBatch(list(reqs), reqs)
        max_tok = max(sum(len(range(r, n, P)) for n in blens) for r in range(P))
        kwargs = []
        for lr, inst in enumerate(instances):
            local_ids = [ids[s + torch.arange(lr, n, P)].tolist() for s, n in zip(starts, blens)]
            kw, run, not_run = pp.prepare_prefill_inputs(batch, (local_ids, max_tok, instances, lr, [True] * len(blens), False, None, None),
                                                         pp.Worker(sp_rank=inst, device="cpu"))
            assert len(run) == len(blens) and not not_run and kw["logical_sp_peer_ranks"] == instances
            assert kw["total_token_num"] <= kw["max_token_num"]
            kwargs.append(kw)
        # every token id appears on exactly one instance, at the striped position
        got = torch.empty_like(ids)
        for lr, kw in enumerate(kwargs):
            off = 0
            for s, n, ln in zip(starts, blens, kw["b_seq_len"].tolist()):
                got[s + torch.arange(lr, n, P)] = kw["input_ids"][off:off + ln]
                off += ln
        assert torch.equal(got, ids)
        # a ring over the prepared metadata only (lengths, start offsets, first global index, number of peers)
        qs, ks, vs = (O.shard_tokens(x, blens, P, True) for x in (q, k, v))
        outs = []
        for lr, kw in enumerate(kwargs):
            o = torch.zeros(kw["total_token_num"], Hq, D); m = torch.full((kw["total_token_num"], Hq), float("-inf")); l = torch.zeros(kw["total_token_num"], Hq)
            for i in range(P):
                src = kwargs[(lr - i) % P]
                O.ring_step(qs[lr], ks[(lr - i) % P], vs[(lr - i) % P], o, m, l, kw["b_start_loc"], kw["b_seq_len"], kw["first_token_global_idx"],
                            src["b_start_loc"], src["b_seq_len"], src["first_token_global_idx"], len(kw["logical_sp_peer_ranks"]))
            outs.append(o)
        ro, _ = O.full_causal_attention(q, k, v, blens)
        o = O.unshard_tokens(outs, blens, P, True)
        assert torch.allclose(o, ro, atol=1e-4, rtol=1e-4)
