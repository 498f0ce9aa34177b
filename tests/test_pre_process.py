"""Worker-side input preparation against the keyword arguments the reference's own
``prepare_prefill_inputs`` / ``prepare_decode_inputs`` produced for the same batches
(tests/golden/pre_process.json, written by tests/golden/make_golden.py)."""
import json
import os

import pytest
import torch

from loongserve_b200 import pre_process as pp

GOLD = os.path.join(os.path.dirname(__file__), "golden", "pre_process.json")


def _same(got, want, key):
    if isinstance(want, dict) and "tensor" in want:
        assert isinstance(got, torch.Tensor), key
        assert str(got.dtype).replace("torch.", "") == want["dtype"], key
        assert got.tolist() == want["tensor"], key
    elif isinstance(want, list):
        assert got is not None and len(got) == len(want), key
        for g, w in zip(got, want):
            _same(g, w, key)
    else:
        assert got == want, key


def _cases(kind):
    with open(GOLD) as f:
        return [c for c in json.load(f) if c["kind"] == kind]


@pytest.mark.parametrize("case", _cases("prefill"), ids=lambda c: "mig" if c["global_input_kvargs"][4] else "plain")
def test_prepare_prefill_inputs_matches_reference(case):
    reqs = {k: pp.InferReq(req_idx=v[0], prompt_len=100, cur_kv_len=v[1]) for k, v in case["requests"].items()}
    batch = pp.InferBatch(list(case["requests"]), reqs)
    gk = (case["input_ids"], *case["global_input_kvargs"])
    kw, run, not_run = pp.prepare_prefill_inputs(batch, gk, pp.Worker(device="cpu"))
    assert [r.req_idx for r in run] == case["run"] and [r.req_idx for r in not_run] == case["not_run"]
    assert set(kw) == set(case["kwargs"])
    for k, want in case["kwargs"].items():
        _same(kw[k], want, k)


@pytest.mark.parametrize("case", _cases("decode"),
                         ids=lambda c: "m%d_r%d" % (c["global_input_kvargs"][2], c["global_input_kvargs"][5]))
def test_prepare_decode_inputs_matches_reference(case):
    reqs = {nm: pp.InferReq(req_idx=10 + i, prompt_len=n, cur_kv_len=n) for i, (nm, n) in enumerate(zip(case["names"], case["lens"]))}
    pp.requests_mapping.clear()
    pp.requests_mapping.update(reqs)                 # the global mapping, as the reference uses it
    try:
        batch = pp.InferBatch(list(case["names"]))
        kw, run, peer_run, not_run = pp.prepare_decode_inputs(batch, tuple(case["global_input_kvargs"]), pp.Worker(device="cpu"))
    finally:
        pp.requests_mapping.clear()
    assert [r.req_idx for r in run] == case["run"] and [r.req_idx for r in peer_run] == case["peer_run"] and not_run == []
    assert [reqs[nm].prompt_len for nm in case["names"]] == case["prompt_len_after"]
    assert set(kw) == set(case["kwargs"])
    for k, want in case["kwargs"].items():
        _same(kw[k], want, k)


def test_tensor_parallel_worker_is_rejected():
    with pytest.raises(NotImplementedError):
        pp.prepare_prefill_inputs(pp.InferBatch([], {}), ([], 0, [0], 0, [], False, None, None), pp.Worker(tp_world_size=2))
