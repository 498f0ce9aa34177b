"""Prefill scheduling search: which new requests run together and on how many instances.

``minimize_prefill_iteration_time`` has the name and the nine positional arguments of the reference's pybind module
(longserve_c_scheduler/src/main.cpp:89-105; call site loongserve/longserve_server/router/manager.py:710-712) and fills the
same two numpy tables in place.  ``plan_prefill_batches`` is the whole planning step of ``_schedule_new_req_list``
(router/manager.py:687-760) in one native call.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import numpy as np

from ._lib import attn as attention_lib, check


def _ptr(a: np.ndarray, dtype) -> ctypes.c_void_p:
    if a.dtype != dtype or not a.flags["C_CONTIGUOUS"]:
        raise TypeError(f"expected a C-contiguous {np.dtype(dtype).name} array, got {a.dtype}")   # pybind's noconvert() does the same
    return ctypes.c_void_p(a.ctypes.data)


def minimize_prefill_iteration_time(num_new_req: int, num_instances: int, min_iteration_times: np.ndarray,
                                    min_iteration_times_index: np.ndarray, req_input_prefix_sum: np.ndarray,
                                    req_input_square_prefix_sum: np.ndarray, inverted_req_input_prefix_sum: np.ndarray,
                                    left_token_prefix_sum: np.ndarray, predictor_parameters: np.ndarray) -> None:
    assert min_iteration_times.shape == (num_new_req + 1, num_instances + 1)
    assert min_iteration_times_index.shape == (num_new_req + 1, num_instances + 1, 2)
    assert predictor_parameters.ndim == 2 and predictor_parameters.shape[1] == 3
    check(attention_lib().esp_sched_minimize_prefill_iteration_time(
        num_new_req, num_instances, _ptr(min_iteration_times, np.float64), _ptr(min_iteration_times_index, np.int32),
        _ptr(req_input_prefix_sum, np.int64), _ptr(req_input_square_prefix_sum, np.int64),
        _ptr(inverted_req_input_prefix_sum, np.float64), _ptr(left_token_prefix_sum, np.int64),
        _ptr(predictor_parameters, np.float64), predictor_parameters.shape[0]), "esp_sched_minimize_prefill_iteration_time")


def plan_prefill_batches(req_tokens: Sequence[int], left_tokens: Sequence[int], predictor_parameters: np.ndarray
                         ) -> Tuple[List[Tuple[slice, slice]], float, float]:
    """req_tokens: lengths of the new requests, longest first; left_tokens: free tokens of the available instances in
    the order the caller sorted them.  Returns ``(batches, total_cost, max_iteration_time)``; every batch is a pair of
    slices (into the request list, into the instance list), last batch first as the reference creates them."""
    rt = np.ascontiguousarray(req_tokens, dtype=np.int64)
    lt = np.ascontiguousarray(left_tokens, dtype=np.int64)
    pp = np.ascontiguousarray(predictor_parameters, dtype=np.float64)
    bs = np.empty(max(len(rt), 1), dtype=np.int32)
    bi = np.empty(max(len(rt), 1), dtype=np.int32)
    nb = ctypes.c_int64(0)
    cost, longest = ctypes.c_double(0.0), ctypes.c_double(0.0)
    check(attention_lib().esp_sched_plan_prefill(len(rt), _ptr(rt, np.int64), len(lt), _ptr(lt, np.int64), _ptr(pp, np.float64),
                                                 pp.shape[0], _ptr(bs, np.int32), _ptr(bi, np.int32), ctypes.byref(nb),
                                                 ctypes.byref(cost), ctypes.byref(longest)), "esp_sched_plan_prefill")
    out, n, m = [], len(rt), None
    m = int(bi[:nb.value].sum())
    for k in range(nb.value):
        out.append((slice(n - int(bs[k]), n), slice(m - int(bi[k]), m)))
        n -= int(bs[k]); m -= int(bi[k])
    return out, cost.value, longest.value
