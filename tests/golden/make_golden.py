"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own code.

Run once in the build container (needs the reference checkout; the GPU box never runs this):

    python tests/golden/make_golden.py /path/to/reference

* Triton kernels of the reference (ring attention step, KV scatter / registration / migration) are
  executed on CPU tensors under Triton's interpreter (TRITON_INTERPRET=1).
* ``torch_att`` and ``init_req_to_token_indexes`` are plain PyTorch and run as they are.
* ``LongServeMemoryManager`` hard-codes device="cuda"; its source is loaded with that literal
  replaced by "cpu" (nothing else is changed, nothing is copied into this repository).

The ring-kernel cases are restricted to shapes where the reference kernel counts each key once:
every q block's visible key range is a multiple of the 128-key tile, or the request has at most
128 local rows (see the note in oracle/esp_oracle.py).
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import importlib.util
import types

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(OUT)))
from loongserve_b200.build import reference_dir  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else reference_dir()
if REF is None:
    sys.exit("usage: make_golden.py /path/to/reference   (or set ESP_REFERENCE_DIR)")


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


ring = load("ref_ring", "loongserve/models/llama/triton_kernel/ring_context_flashattention_nopad.py")
carkv = load("ref_carkv", "loongserve/models/llama/triton_kernel/copy_and_register_kv.py")
mig = load("ref_mig", "loongserve/models/llama/triton_kernel/decoding_stage_migration.py")
dcopy = load("ref_dcopy", "loongserve/common/basemodel/triton_kernel/destindex_copy_kv.py")
idx2req = load("ref_idx2req", "loongserve/common/basemodel/triton_kernel/copy_kv_index_to_req.py")
infer_utils = load("ref_infer_utils", "loongserve/common/infer_utils.py")


def i32(x):
    return torch.tensor(x, dtype=torch.int32)


def shard(x, lens, P, striped):
    outs = [[] for _ in range(P)]
    s = 0
    for L in lens:
        seq = x[s:s + L]
        for r in range(P):
            if striped:
                outs[r].append(seq[r::P])
            else:
                per = (L + P - 1) // P
                outs[r].append(seq[min(L, r * per):min(L, (r + 1) * per)])
        s += L
    return [torch.cat(o, 0).contiguous() for o in outs]


def ring_case(name, lens, P, striped, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    q = torch.randn(T, Hq, D, generator=g).half()
    k = torch.randn(T, Hkv, D, generator=g).half()
    v = torch.randn(T, Hkv, D, generator=g).half()
    qs, ks, vs = shard(q, lens, P, striped), shard(k, lens, P, striped), shard(v, lens, P, striped)
    llen = [[(max(0, (L - r + P - 1) // P) if striped else
              (min(L, (r + 1) * ((L + P - 1) // P)) - min(L, r * ((L + P - 1) // P)))) for L in lens] for r in range(P)]
    first = [[(r if striped else min(L, r * ((L + P - 1) // P))) for L in lens] for r in range(P)]
    stride = P if striped else 1
    out = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), lens=np.array(lens, np.int32),
               P=np.int32(P), striped=np.int32(striped))
    for r in range(P):
        Tq = qs[r].shape[0]
        o = torch.zeros_like(qs[r])
        m = torch.full((Tq, Hq), -float("inf"))
        l = torch.zeros(Tq, Hq)
        q_len = i32(llen[r]); q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
        for i in range(P):
            src = (r - i) % P
            kv_len = i32(llen[src]); kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
            ring.context_attention_fwd(qs[r], ks[src], vs[src], o, q_start, q_len, i32(first[r]),
                                       kv_start, kv_len, i32(first[src]), stride, int(q_len.max()), m, l)
            out[f"o_r{r}_s{i}"] = o.numpy().copy()
            out[f"m_r{r}_s{i}"] = m.numpy().copy()
            out[f"l_r{r}_s{i}"] = l.numpy().copy()
    np.savez_compressed(os.path.join(OUT, name), **out)
    print("wrote", name)


def torch_att_case():
    g = torch.Generator().manual_seed(11)
    lens = [300, 77, 205]
    T, Hq, Hkv, D = sum(lens), 4, 2, 128
    q = torch.randn(T, Hq, D, generator=g).half()
    k = torch.randn(T, Hkv, D, generator=g).half()
    v = torch.randn(T, Hkv, D, generator=g).half()
    o = ring.torch_att(q.float(), k.float(), v.float(), torch.tensor(lens))
    np.savez_compressed(os.path.join(OUT, "torch_att_varlen.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        lens=np.array(lens, np.int32), o=o.numpy())
    # the reference self-test's value distribution (ring_context_flashattention_nopad.py:344-346)
    g = torch.Generator().manual_seed(0)
    lens = [211, 340]
    T, Hq, Hkv, D = sum(lens), 6, 2, 64
    q = (torch.randn(T, Hq, D, generator=g) * 0.2 + 0.1).half()
    k = (torch.randn(T, Hkv, D, generator=g) * 0.2 + 0.4).half()
    v = (torch.randn(T, Hkv, D, generator=g) * 0.2 + 0.3).half()
    o = ring.torch_att(q.float(), k.float(), v.float(), torch.tensor(lens))
    np.savez_compressed(os.path.join(OUT, "torch_att_selftest_dist.npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        lens=np.array(lens, np.int32), o=o.numpy())
    print("wrote torch_att cases")


def kv_cases():
    g = torch.Generator().manual_seed(5)
    H2, D = 4, 16
    # destindex_copy_kv
    K = torch.randn(37, H2, D, generator=g).half()
    dest = torch.randperm(64, generator=g)[:37].to(torch.int32)
    Out = torch.zeros(64, H2, D).half()
    dcopy.destindex_copy_kv(K, dest, Out)
    res = dict(dc_K=K.numpy(), dc_dest=dest.numpy(), dc_out=Out.numpy())

    # pre_copy_and_register_kv + destindex_copy_and_register_kv, over a whole ring pass (P = 3)
    P, B = 3, 3
    lens = [17, 5, 300]
    cache_begin = i32([3, 0, 40]); cache_end = i32([12, 5, 299])
    b_req_idx = i32([2, 0, 1])
    n_keep = int((cache_end - cache_begin).sum())
    pool = torch.zeros(400, H2, D).half()
    mem_index = torch.randperm(400, generator=g)[:n_keep].to(torch.int64)
    req_to_tok = torch.full((4, 320), 2147483647, dtype=torch.int32)
    cur_idx = torch.zeros(B, dtype=torch.int32)
    used = 0
    res.update(cr_lens=np.array(lens, np.int32), cr_cache_begin=cache_begin.numpy(), cr_cache_end=cache_end.numpy(),
               cr_b_req_idx=b_req_idx.numpy(), cr_mem_index=mem_index.numpy(), cr_P=np.int32(P))
    for r in range(P):
        llen = [max(0, (L - r + P - 1) // P) for L in lens]
        kv = torch.randn(sum(llen) + 2, H2, D, generator=g).half()
        kv_len = i32(llen); kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
        kvf = i32([r] * B)
        rb, re, nl = carkv.pre_copy_and_register_kv(cache_begin, cache_end, kvf, P)
        nls = torch.cumsum(nl, 0, dtype=torch.int64)
        carkv.destindex_copy_and_register_kv(B, nl, rb, re, nls, kv, kv_start, cur_idx, mem_index, pool,
                                             req_to_tok, b_req_idx, used, max(llen) + 1, True)
        used += int(nls[-1])
        cur_idx += nl
        res.update({f"cr_kv_{r}": kv.numpy(), f"cr_rb_{r}": rb.numpy(), f"cr_re_{r}": re.numpy(),
                    f"cr_nl_{r}": nl.numpy()})
    res.update(cr_pool=pool.numpy(), cr_req_to_tok=req_to_tok.numpy(), cr_cur_idx=cur_idx.numpy())

    # copy_kv_index_to_req
    rt = torch.full((5, 40), 2147483647, dtype=torch.int32)
    b_req = i32([3, 1, 4]); b_len = i32([7, 40, 1]); memidx = i32([11, 22, 33])
    idx2req.copy_kv_index_to_req(rt, b_req, b_len, memidx)
    res.update(ci_b_req=b_req.numpy(), ci_b_len=b_len.numpy(), ci_memidx=memidx.numpy(), ci_out=rt.numpy())

    # init_req_to_token_indexes
    rt = torch.full((5, 40), 2147483647, dtype=torch.int32)
    b_req = i32([2, 0, 4]); b_len = i32([9, 0, 31])
    alloc = torch.randperm(100, generator=g)[:40].to(torch.int64)
    infer_utils.init_req_to_token_indexes(rt, b_req, b_len, alloc)
    res.update(ii_b_req=b_req.numpy(), ii_b_len=b_len.numpy(), ii_alloc=alloc.numpy(), ii_out=rt.numpy())

    # decode-stage migration, sender then receiver
    L, S = 3, 50
    kvc = torch.randn(L, S, H2, D, generator=g).half()
    rt = torch.full((4, 30), 2147483647, dtype=torch.int32)
    lens_s = [12, 30, 4]
    perm = torch.randperm(S, generator=g).to(torch.int32)
    o = 0
    for rid, n in zip([1, 3, 0], lens_s):
        rt[rid, :n] = perm[o:o + n]; o += n
    mem_state = torch.zeros(S, dtype=torch.int32); mem_state[perm[:o].long()] = 1
    req_ids = i32([1, 3, 0]); ntok = i32([5, 0, 4]); b_len = i32(lens_s)
    send = torch.zeros(L, int(ntok.sum()), H2, D).half()
    res.update(mg_kvc=kvc.numpy(), mg_rt=rt.numpy().copy(), mg_mem_state_in=mem_state.numpy().copy(),
               mg_req_ids=req_ids.numpy(), mg_ntok=ntok.numpy(), mg_b_len=b_len.numpy())
    mig.decoding_stage_migration_sender_kernel(send, rt, mem_state, kvc, req_ids, ntok, b_len)
    res.update(mg_send=send.numpy(), mg_mem_state_out=mem_state.numpy())
    kvc2 = torch.zeros(L, 40, H2, D).half()
    rt2 = torch.full((4, 30), 2147483647, dtype=torch.int32)
    alloc = torch.randperm(40, generator=g)[: int(ntok.sum())].to(torch.int64)
    b_len2 = i32([2, 7, 0])
    mig.decoding_stage_migration_receiver_kernel(send, rt2, kvc2, alloc, req_ids, ntok, b_len2)
    res.update(mg_alloc=alloc.numpy(), mg_b_len2=b_len2.numpy(), mg_kvc2=kvc2.numpy(), mg_rt2=rt2.numpy())
    np.savez_compressed(os.path.join(OUT, "kv_ops.npz"), **res)
    print("wrote kv_ops.npz")


def mem_manager_case():
    src = open(os.path.join(REF, "loongserve/common/longserve_mem_manager.py")).read()
    src = src.replace('device="cuda"', 'device="cpu"')
    src = src.replace("from loongserve.utils.log_utils import init_logger", "import logging\ninit_logger = logging.getLogger")
    mod = types.ModuleType("ref_mem_manager")
    exec(compile(src, "ref_mem_manager", "exec"), mod.__dict__)
    mm = mod.LongServeMemoryManager(64, torch.float16, 2, 8, 1)
    trace = []
    a = mm.alloc(5); trace.append(("alloc5", a.numpy().copy(), mm.can_use_mem_size))
    b = mm.alloc_contiguous(7); trace.append(("contig7", b[0].numpy().copy(), mm.can_use_mem_size))
    mm.free(a[1:4]); trace.append(("free_a1_4", mm.mem_state.numpy().copy(), mm.can_use_mem_size))
    c = mm.alloc(6); trace.append(("alloc6", c.numpy().copy(), mm.can_use_mem_size))
    d = mm.alloc_contiguous(4); trace.append(("contig4", d[0].numpy().copy(), mm.can_use_mem_size))
    mm.add_refs(c[:2]); trace.append(("addref", mm.mem_state.numpy().copy(), mm.can_use_mem_size))
    mm.free(c); trace.append(("free_c", mm.mem_state.numpy().copy(), mm.can_use_mem_size))
    e = mm.alloc_contiguous(60); trace.append(("contig60", np.array([-1 if e is None else 0]), mm.can_use_mem_size))
    out = {}
    for i, (nm, arr, free) in enumerate(trace):
        out[f"t{i}_{nm}"] = np.asarray(arr)
        out[f"t{i}_free"] = np.int64(free)
    np.savez_compressed(os.path.join(OUT, "mem_manager.npz"), **out)
    print("wrote mem_manager.npz")


def _plain(x):
    if isinstance(x, torch.Tensor):
        return {"tensor": x.tolist(), "dtype": str(x.dtype).replace("torch.", "")}
    if isinstance(x, (list, tuple)):
        return [_plain(y) for y in x]
    if isinstance(x, (np.integer,)):
        return int(x)
    return x


def pre_process_case():
    """Runs the reference's prepare_prefill_inputs / prepare_decode_inputs on CPU: the module is loaded from its
    source text with the 'cuda' device literals replaced by 'cpu' and its three project imports replaced by small
    stand-ins for the request record, the batch and the status enum (nothing else changes)."""
    import json
    src = open(os.path.join(REF, "loongserve/longserve_server/router/model_infer/pre_process.py")).read()
    src = src.replace("device='cuda'", "device='cpu'").replace('device="cuda"', 'device="cpu"')
    src = src.replace("from .infer_batch import requests_mapping, InferReq, InferBatch", "")
    src = src.replace("from loongserve.longserve_server.io_struct import ReqRunStatus", "")
    src = src.replace("from loongserve.utils.infer_utils import calculate_time", "")
    mod = types.ModuleType("ref_pre_process")

    class ReqRunStatus:
        RUNNING = 1

    class InferReq:
        def __init__(self, req_idx, prompt_len, cur_kv_len):
            self.req_idx, self.prompt_len, self.cur_kv_len, self.req_status = req_idx, prompt_len, cur_kv_len, ReqRunStatus.RUNNING

    class InferBatch:
        def __init__(self, ids):
            self.request_ids = ids

        def __len__(self):
            return len(self.request_ids)

    class W:
        tp_rank, tp_world_size, sp_rank = 0, 1, 0

    mod.__dict__.update(requests_mapping={}, InferReq=InferReq, InferBatch=InferBatch, ReqRunStatus=ReqRunStatus)
    exec(compile(src, "ref_pre_process", "exec"), mod.__dict__)
    rm = mod.requests_mapping
    cases = []
    rng = np.random.RandomState(11)
    # ---- prefill: request 'c' was prefilled before (skipped); request 'd' has no token on this instance
    for need_mig in (False, True):
        rm.clear()
        spec = {"a": (5, 0, 7), "b": (2, 0, 1), "c": (9, 33, 4), "d": (0, 0, 0), "e": (7, 0, 12)}      # req_idx, cur_kv_len, local tokens
        for k, (ri, ckl, n) in spec.items():
            rm[k] = InferReq(ri, 100, ckl)
        ids = [rng.randint(0, 32000, size=n).tolist() for (_, _, n) in spec.values()]
        gk = (ids, 16, [3, 1, 2], 1, [True] * 5, need_mig, [0, 4, 0, 9] if need_mig else None, [10, 4, 3, 40] if need_mig else None)
        kw, run, not_run = mod.prepare_prefill_inputs(InferBatch(list(spec)), gk, W)
        cases.append(dict(kind="prefill", requests={k: list(v) for k, v in spec.items()}, input_ids=ids, global_input_kvargs=_plain(list(gk[1:])),
                          kwargs={k: _plain(v) for k, v in kw.items()}, run=[r.req_idx for r in run], not_run=[r.req_idx for r in not_run]))
    # ---- prefill with nothing to run
    rm.clear(); rm["z"] = InferReq(1, 50, 50)
    kw, run, not_run = mod.prepare_prefill_inputs(InferBatch(["z"]), ([[1, 2]], 8, [0, 1], 0, [True], False, None, None), W)
    cases.append(dict(kind="prefill", requests={"z": [1, 50, 2]}, input_ids=[[1, 2]], global_input_kvargs=_plain([8, [0, 1], 0, [True], False, None, None]),
                      kwargs={k: _plain(v) for k, v in kw.items()}, run=[r.req_idx for r in run], not_run=[r.req_idx for r in not_run]))
    # ---- decode: 4 instances in the order [2, 0, 3, 1], masters = logical ranks 0..1 (or only 0), every logical rank's view
    for num_masters, sizes in ((2, [2, 4]), (1, [6]), (3, [1, 2, 3])):
        for lr in range(4):
            rm.clear()
            names = ["r%d" % i for i in range(6)]
            lens = [40, 17, 300, 5, 64, 128]
            bounds = np.concatenate([[0], np.cumsum(sizes)])
            lo, hi = (bounds[lr], bounds[lr + 1]) if lr < num_masters else (6, 6)
            for i, nm in enumerate(names):
                rm[nm] = InferReq(10 + i, lens[i], lens[i])
            n_own = int(hi - lo)
            ids = rng.randint(0, 32000, size=n_own).tolist()
            first = [lens[i] * 4 + lr for i in range(lo, hi)]
            gk = (ids, first, num_masters, sizes, [2, 0, 3, 1], lr)
            kw, run, peer_run, not_run = mod.prepare_decode_inputs(InferBatch(names), gk, W)
            cases.append(dict(kind="decode", names=names, lens=lens, global_input_kvargs=_plain(list(gk)),
                              kwargs={k: _plain(v) for k, v in kw.items()}, run=[r.req_idx for r in run],
                              peer_run=[r.req_idx for r in peer_run], not_run=[r.req_idx for r in not_run],
                              prompt_len_after=[rm[nm].prompt_len for nm in names]))
    with open(os.path.join(OUT, "pre_process.json"), "w") as f:
        json.dump(cases, f, indent=0)
    print("wrote pre_process.json,", len(cases), "cases")


def scheduler_inputs(seed, R, I, tight):
    """Seeded inputs of the prefill scheduling search, prepared as router/manager.py:691-707 does."""
    rng = np.random.RandomState(seed)
    lens = np.sort(np.round(np.exp(rng.uniform(np.log(64), np.log(200000), size=R))).astype(np.int64))[::-1].copy()
    if tight == "bimodal":                            # a few very long requests and many short ones: plans with several batches
        lens = np.sort(np.concatenate([rng.randint(100000, 200000, size=max(R // 6, 1)), rng.randint(50, 400, size=R - max(R // 6, 1))]).astype(np.int64))[::-1].copy()
        tight = False
    cap = 250000
    used = np.sort(rng.randint(0, cap // 2 if not tight else cap - 20000, size=I))
    room = (cap - used).astype(np.int64)
    if room.sum() < lens.sum():                       # the router only calls the search when everything fits
        lens = np.maximum(lens * room.sum() // (lens.sum() + 1), 1)
    abc = np.full((I + 1, 3), np.nan)
    for u in range(1, I + 1):
        abc[u] = (0.02 + 0.004 * u, 4.0e-5 / u * (1 + 0.05 * u), 2.5e-10 / u * (1 + 0.03 * u))
    return lens, room, abc


def scheduler_case():
    """Runs the reference's compiled search (oracle/_ref/longserve_c_scheduler.so, built by oracle/Makefile from the
    reference's single source file)."""
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(OUT)), "oracle", "_ref"))
    import longserve_c_scheduler as ref
    out = {}
    shapes = [(1, 1, False), (3, 2, False), (6, 4, False), (12, 8, False), (24, 8, True), (9, 3, True), (40, 8, False), (16, 5, True),
              (12, 8, "bimodal"), (30, 6, "bimodal"), (7, 4, "bimodal")]
    for k, (R, I, tight) in enumerate(shapes):
        lens, room, abc = scheduler_inputs(100 + k, R, I, tight)
        best = np.full((R + 1, I + 1), np.inf)
        choice = np.full((R + 1, I + 1, 2), -1, dtype=np.int32)
        ref.minimize_prefill_iteration_time(R, I, best, choice, np.cumsum(lens), np.cumsum(lens ** 2), np.cumsum(1.0 / lens.astype(np.float64)),
                                            np.cumsum(room), abc)
        out[f"c{k}_lens"], out[f"c{k}_room"], out[f"c{k}_abc"], out[f"c{k}_best"], out[f"c{k}_choice"] = lens, room, abc, best, choice
    out["n"] = np.int64(len(shapes))
    np.savez_compressed(os.path.join(OUT, "scheduler_dp.npz"), **out)
    print("wrote scheduler_dp.npz")


if __name__ == "__main__":
    only = sys.argv[2:]
    if only:                         # e.g. `make_golden.py /path/to/reference pre_process`
        with torch.inference_mode():
            for name in only:
                globals()[name + "_case"]()
        sys.exit(0)
    with torch.inference_mode():
        ring_case("ring_ref_contig_p2.npz", [512], 2, False, 2, 1, 128, 1)
        ring_case("ring_ref_striped_p4.npz", [509, 203], 4, True, 2, 1, 128, 2)
        ring_case("ring_ref_varlen_p8.npz", [97, 128, 31, 8], 8, False, 4, 2, 32, 3)
        torch_att_case()
        kv_cases()
        mem_manager_case()
        pre_process_case()
        scheduler_case()
