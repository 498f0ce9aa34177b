"""Make the reference's own import statements resolve to this package.

The reference reaches the hot path through plain imports
(loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:6-15, loongserve/models/llama/longserve_model.py:6,17-21,591,
loongserve/longserve_server/router/manager.py:29).  ``install()`` registers modules under exactly those names, so an unmodified
``longserve_transformer_layer_infer.py`` picks up the B200 kernels:

    import loongserve_b200.dropin as dropin
    dropin.install()            # before the reference's model modules are imported

Three top-level extension modules are replaced whole (``rnccl``, ``longserve_cuda_kernels``, ``longserve_c_scheduler``).  Inside the
``loongserve`` package only the listed leaf modules are replaced; when the real package is importable its other modules are
left alone, and when it is not (this repository's tests) empty parent packages are created so that the imports still work.
``uninstall()`` restores what was there before.
"""
from __future__ import annotations

import importlib
import sys
import types
from typing import Dict, List, Tuple

_saved: List[Tuple[str, object]] = []
_MISSING = object()


def _module(name: str, **attrs) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    m.__dict__["__esp_dropin__"] = True
    return m


def alias_table() -> Dict[str, types.ModuleType]:
    """Reference module path -> module object exporting the names the reference imports from it."""
    from . import context_attention, flash_decoding, kv_ops, layer_ops, mem_manager, pre_process, rnccl, scheduler
    tk = "loongserve.models.llama.triton_kernel."
    bk = "loongserve.common.basemodel.triton_kernel."
    return {
        "rnccl": _module("rnccl", get_nccl_unique_id=rnccl.get_nccl_unique_id, RNCCLComm=rnccl.RNCCLComm),
        "longserve_cuda_kernels": _module(
            "longserve_cuda_kernels", flash_decoding_stage1=flash_decoding.flash_decoding_stage1,
            flash_decoding_stage2=flash_decoding.flash_decoding_stage2, rms_norm=layer_ops.rms_norm, rotary_emb=layer_ops.rotary_emb,
            silu_and_mul_inplace=layer_ops.silu_and_mul_inplace, ffn_block=layer_ops.ffn_block),
        "longserve_c_scheduler": _module("longserve_c_scheduler",
                                         minimize_prefill_iteration_time=scheduler.minimize_prefill_iteration_time),
        tk + "ring_context_flashattention_nopad": _module(tk + "ring_context_flashattention_nopad",
                                                          context_attention_fwd=context_attention.context_attention_fwd),
        tk + "longserve_flash_decoding": _module(
            tk + "longserve_flash_decoding",
            longserve_token_decode_attention_flash_decoding=flash_decoding.longserve_token_decode_attention_flash_decoding),
        tk + "longserve_flash_decoding_stage1": _module(tk + "longserve_flash_decoding_stage1",
                                                        longserve_flash_decode_stage1=flash_decoding.longserve_flash_decode_stage1),
        tk + "longserve_flash_decoding_stage2": _module(tk + "longserve_flash_decoding_stage2",
                                                        longserve_flash_decode_stage2=flash_decoding.longserve_flash_decode_stage2),
        tk + "copy_and_register_kv": _module(tk + "copy_and_register_kv", pre_copy_and_register_kv=kv_ops.pre_copy_and_register_kv,
                                             destindex_copy_and_register_kv=kv_ops.destindex_copy_and_register_kv),
        tk + "decoding_stage_migration": _module(
            tk + "decoding_stage_migration", decoding_stage_migration_sender_kernel=kv_ops.decoding_stage_migration_sender_kernel,
            decoding_stage_migration_receiver_kernel=kv_ops.decoding_stage_migration_receiver_kernel),
        bk + "destindex_copy_kv": _module(bk + "destindex_copy_kv", destindex_copy_kv=kv_ops.destindex_copy_kv),
        bk + "copy_kv_index_to_req": _module(bk + "copy_kv_index_to_req", copy_kv_index_to_req=kv_ops.copy_kv_index_to_req),
        "loongserve.common.longserve_mem_manager": _module("loongserve.common.longserve_mem_manager",
                                                           LongServeMemoryManager=mem_manager.LongServeMemoryManager),
        "loongserve.common.longserve_req_manager": _module("loongserve.common.longserve_req_manager",
                                                           LongServeReqManager=mem_manager.LongServeReqManager),
    }


# Names replaced INSIDE a reference module that also holds things outside the path (the module itself stays).
def patch_table():
    from . import kv_ops, pre_process
    return {
        "loongserve.common.infer_utils": {"init_req_to_token_indexes": kv_ops.init_req_to_token_indexes},
        "loongserve.longserve_server.router.model_infer.pre_process": {
            "prepare_prefill_inputs": pre_process.prepare_prefill_inputs, "prepare_decode_inputs": pre_process.prepare_decode_inputs},
    }


def _ensure_parent(path: str):
    """Import (or, when the reference package is absent, create) every parent package of ``path``; returns the direct parent."""
    parts = path.split(".")[:-1]
    parent = None
    for i in range(len(parts)):
        name = ".".join(parts[:i + 1])
        mod = sys.modules.get(name)
        if mod is None:
            try:
                mod = importlib.import_module(name)
            except Exception:
                mod = _module(name, __path__=[])
                _saved.append((name, _MISSING))
                sys.modules[name] = mod
                if parent is not None:
                    setattr(parent, parts[i], mod)
        parent = mod
    return parent


def install(patch_partial: bool = True) -> List[str]:
    """Register the aliases.  Returns the module paths now served by this package."""
    if _saved:
        return [n for n, _ in _saved]
    done = []
    for path, mod in alias_table().items():
        parent = _ensure_parent(path) if "." in path else None
        _saved.append((path, sys.modules.get(path, _MISSING)))
        sys.modules[path] = mod
        if parent is not None:
            setattr(parent, path.rsplit(".", 1)[1], mod)
        done.append(path)
    if patch_partial:
        for path, names in patch_table().items():
            try:
                target = importlib.import_module(path)
            except Exception:
                parent = _ensure_parent(path)
                target = _module(path)
                _saved.append((path, _MISSING))
                sys.modules[path] = target
                setattr(parent, path.rsplit(".", 1)[1], target)
            for k, v in names.items():
                _saved.append((path + ":" + k, getattr(target, k, _MISSING)))
                setattr(target, k, v)
            done.append(path)
    return done


def uninstall() -> None:
    while _saved:
        key, old = _saved.pop()
        if ":" in key:
            path, attr = key.split(":")
            target = sys.modules.get(path)
            if target is not None:
                if old is _MISSING:
                    if hasattr(target, attr):
                        delattr(target, attr)
                else:
                    setattr(target, attr, old)
        elif old is _MISSING:
            sys.modules.pop(key, None)
        else:
            sys.modules[key] = old
