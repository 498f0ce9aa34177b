"""The reference's own Triton ring kernel, compiled by the installed Triton for this GPU, run next to esp_prefill_step.

The reference kernel is fp16-only (loongserve/models/llama/triton_kernel/ring_context_flashattention_nopad.py:138,167,183)
and exact only where every visible key range is a multiple of its 128-key block: its masked tail loop starts 128 keys before
the end of the range (:114,143) and so counts the keys of a ragged tail twice.  One fp16 sequence of 16384 tokens on a
ring of four, emulated on one GPU:

* contiguous shards (4096 tokens each): every visible range is a multiple of 128, so both kernels must agree after every
  ring step -- o directly, (m, l) through the log-sum-exp they encode, because this kernel keeps a lazily updated maximum
  while the reference keeps the exact one;
* striped shards (the reference's own placement, token t on shard t mod 4): blocks of higher-numbered shards are visible
  up to one key short of a block boundary, the ragged case.  Here this package's result must match fp32 attention; how far
  the reference kernel is from fp32 on the same inputs is recorded, not asserted.

Needs the reference's Python package: a checkout named by ESP_REFERENCE_DIR (or next to this repository), or an
installed copy under baseline/_ref.  Skipped when neither is there or when Triton cannot build the kernel here."""
import importlib.util
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = os.path.join("loongserve", "models", "llama", "triton_kernel", "ring_context_flashattention_nopad.py")


def _reference_kernel():
    from loongserve_b200.build import reference_dir
    for base in (reference_dir(), os.path.join(ROOT, "baseline", "_ref")):
        if base and os.path.exists(os.path.join(base, REL)):
            spec = importlib.util.spec_from_file_location("ref_ring_kernel", os.path.join(base, REL))
            mod = importlib.util.module_from_spec(spec)
            try:
                spec.loader.exec_module(mod)
            except Exception as e:                       # noqa: BLE001
                pytest.skip(f"the reference kernel module does not import here: {type(e).__name__}: {e}")
            return mod
    pytest.skip("reference package not present (ESP_REFERENCE_DIR, a sibling checkout, or baseline/_ref)")


def _fp32_causal(q, k, v, rows_per_chunk=2048):
    """Full causal attention in fp32 on the device, head by head and in row chunks: (o, lse)."""
    T, Hh, D = q.shape
    o = torch.empty(T, Hh, D, device=q.device); lse = torch.empty(T, Hh, device=q.device)
    pos = torch.arange(T, device=q.device)
    for h in range(Hh):
        kh, vh = k[:, h].float(), v[:, h].float()
        for r0 in range(0, T, rows_per_chunk):
            r1 = min(T, r0 + rows_per_chunk)
            sc = (q[r0:r1, h].float() @ kh[:r1].t()) * (D ** -0.5)
            sc.masked_fill_(pos[:r1][None, :] > pos[r0:r1][:, None], float("-inf"))
            lse[r0:r1, h] = torch.logsumexp(sc, 1)
            o[r0:r1, h] = torch.softmax(sc, 1) @ vh[:r1]
    return o, lse


def test_reference_triton_ring_kernel_step_by_step():
    assert os.environ.get("TRITON_INTERPRET", "0") != "1"
    from loongserve_b200 import context_attention as ca
    from loongserve_b200 import ring
    ref = _reference_kernel()
    dev = "cuda"
    P, T, Hq, Hkv, D = 4, 16384, 8, 8, 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, Hq, D, generator=g).to(torch.float16).to(dev)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.float16).to(dev)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.float16).to(dev)
    full_o, full_lse = _fp32_causal(q, k, v)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = {"reference": [], "ours": []}
    first_call = [True]
    report = {}
    for striped in (False, True):
        local_len, first, stride = ring.shard_lengths([T], P, striped)
        Tl = T // P
        shard = (lambda x, r: x[r::P].contiguous()) if striped else (lambda x, r: x[r * Tl:(r + 1) * Tl].contiguous())
        qs, ks, vs = ([shard(x, r) for r in range(P)] for x in (q, k, v))
        metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], dev) for r in range(P)]
        worst = {"step_o": 0.0, "step_lse": 0.0, "ours_o": 0.0, "ours_lse": 0.0, "ref_o": 0.0, "ref_lse": 0.0}
        for r in range(P):
            st = {name: (torch.zeros(Tl, Hq, D, dtype=torch.float16, device=dev), torch.full((Tl, Hq), float("-inf"), device=dev),
                         torch.zeros(Tl, Hq, device=dev)) for name in ("reference", "ours")}
            for i in range(P):
                src = (r - i) % P
                args = (metas[r].start_loc, metas[r].seq_len, metas[r].first_idx, metas[src].start_loc, metas[src].seq_len,
                        metas[src].first_idx, stride, Tl)
                for name, fn in (("reference", ref.context_attention_fwd), ("ours", ca.context_attention_fwd)):
                    o, m, l = st[name]
                    try:
                        e0.record()
                        fn(qs[r], ks[src], vs[src], o, *args, m, l)
                        e1.record()
                        torch.cuda.synchronize()
                    except Exception as e:               # noqa: BLE001
                        if name == "reference" and first_call[0]:
                            pytest.skip(f"Triton could not build or launch the reference kernel here: {type(e).__name__}: {e}")
                        raise
                    if name == "ours" or not first_call[0]:      # the reference's first call includes Triton's compilation
                        times[name].append(e0.elapsed_time(e1))
                    if name == "reference":
                        first_call[0] = False
                if not striped:
                    (o_r, m_r, l_r), (o_o, m_o, l_o) = st["reference"], st["ours"]
                    lse_r, lse_o = ca.attention_lse(m_r, l_r), ca.attention_lse(m_o, l_o)
                    fin = torch.isfinite(lse_r)
                    assert torch.equal(fin, torch.isfinite(lse_o)), f"rank {r} step {i}: different rows have seen keys"
                    do = (o_o.float() - o_r.float()).abs()
                    worst["step_o"] = max(worst["step_o"], float(do.max()))
                    worst["step_lse"] = max(worst["step_lse"], float((lse_o[fin] - lse_r[fin]).abs().max()))
                    assert bool((do <= 2e-2 + 1e-2 * o_r.float().abs()).all()), f"rank {r} step {i}: o differs by {float(do.max())}"
                    assert torch.allclose(lse_o[fin], lse_r[fin], atol=1e-3, rtol=1e-3), f"rank {r} step {i}: lse differs"
            # after the last step: both against fp32 attention of the whole sequence
            want_o, want_lse = shard(full_o, r), shard(full_lse, r)
            for name in ("ours", "reference"):
                o, m, l = st[name]
                key = "ours" if name == "ours" else "ref"
                worst[key + "_o"] = max(worst[key + "_o"], float((o.float() - want_o).abs().max()))
                worst[key + "_lse"] = max(worst[key + "_lse"], float((ca.attention_lse(m, l) - want_lse).abs().max()))
            o, m, l = st["ours"]
            assert bool(((o.float() - want_o).abs() <= 2e-2 + 1e-2 * want_o.abs()).all()), f"rank {r}: ours differs from fp32"
            assert torch.allclose(ca.attention_lse(m, l), want_lse, atol=1e-3, rtol=1e-3), f"rank {r}: our lse differs from fp32"
            if not striped:
                o, m, l = st["reference"]
                assert bool(((o.float() - want_o).abs() <= 2e-2 + 1e-2 * want_o.abs()).all()), f"rank {r}: the reference differs from fp32"
        report["striped" if striped else "contiguous"] = worst
    assert ca.device_status()[0] == 0
    # medians: a few of the reference's calls include a Triton re-specialisation (an integer argument becoming 1)
    tr = sorted(times["reference"])[len(times["reference"]) // 2]; to = sorted(times["ours"])[len(times["ours"]) // 2]
    c, s_ = report["contiguous"], report["striped"]
    line = (f"reference Triton kernel vs esp_prefill_step on one B200, fp16, {T} tokens x {Hq} heads x {D}, ring of {P} emulated: "
            f"median ms per ring step reference {tr:.3f}, ours {to:.3f} (x{tr / to:.1f}). "
            f"Contiguous shards: max step-by-step |o diff| {c['step_o']:.2e}, |lse diff| {c['step_lse']:.2e}; vs fp32: ours {c['ours_o']:.2e}, "
            f"reference {c['ref_o']:.2e}. Striped shards (ragged visible ranges) vs fp32: ours |o| {s_['ours_o']:.2e} |lse| {s_['ours_lse']:.2e}, "
            f"reference |o| {s_['ref_o']:.2e} |lse| {s_['ref_lse']:.2e}")
    print(line)
    out_dir = os.environ.get("ESP_TEST_REPORT_DIR")            # where to leave the line as a file, if anywhere
    if out_dir and os.path.isdir(out_dir):
        with open(os.path.join(out_dir, "reference_triton_vs_ours.txt"), "w") as f:
            f.write(line + "\n")
