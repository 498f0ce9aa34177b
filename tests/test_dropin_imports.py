"""After ``dropin.install()`` the import statements of the reference's layer-infer and model modules
(longserve_transformer_layer_infer.py:6-15, longserve_model.py:6,17-21,591, router/manager.py:29) resolve to this package."""
import importlib
import sys

import pytest

from loongserve_b200 import dropin

REFERENCE_IMPORTS = """
import rnccl
import longserve_cuda_kernels
import longserve_c_scheduler
from loongserve.common.basemodel.triton_kernel.destindex_copy_kv import destindex_copy_kv
from loongserve.models.llama.triton_kernel.ring_context_flashattention_nopad import context_attention_fwd
from loongserve.models.llama.triton_kernel.longserve_flash_decoding import longserve_token_decode_attention_flash_decoding
from loongserve.models.llama.triton_kernel.longserve_flash_decoding_stage1 import longserve_flash_decode_stage1
from loongserve.models.llama.triton_kernel.longserve_flash_decoding_stage2 import longserve_flash_decode_stage2
from loongserve.models.llama.triton_kernel.copy_and_register_kv import pre_copy_and_register_kv, destindex_copy_and_register_kv
from loongserve.models.llama.triton_kernel.decoding_stage_migration import decoding_stage_migration_sender_kernel, decoding_stage_migration_receiver_kernel
from loongserve.common.longserve_mem_manager import LongServeMemoryManager
from loongserve.common.longserve_req_manager import LongServeReqManager
from loongserve.common.infer_utils import init_req_to_token_indexes
from loongserve.common.basemodel.triton_kernel.copy_kv_index_to_req import copy_kv_index_to_req
from loongserve.longserve_server.router.model_infer.pre_process import prepare_prefill_inputs, prepare_decode_inputs
"""


@pytest.fixture
def installed():
    before = set(sys.modules)
    served = dropin.install()
    yield served
    dropin.uninstall()
    for name in set(sys.modules) - before:
        if name.split(".")[0] in ("loongserve", "rnccl", "longserve_cuda_kernels", "longserve_c_scheduler"):
            sys.modules.pop(name, None)


def test_reference_import_lines_resolve_to_this_package(installed):
    ns = {}
    exec(REFERENCE_IMPORTS, ns)
    from loongserve_b200 import context_attention, flash_decoding, kv_ops, layer_ops, mem_manager, pre_process, scheduler
    from loongserve_b200 import rnccl as our_rnccl
    assert ns["context_attention_fwd"] is context_attention.context_attention_fwd
    assert ns["rnccl"].RNCCLComm is our_rnccl.RNCCLComm and ns["rnccl"].get_nccl_unique_id is our_rnccl.get_nccl_unique_id
    k = ns["longserve_cuda_kernels"]
    assert k.flash_decoding_stage1 is flash_decoding.flash_decoding_stage1 and k.flash_decoding_stage2 is flash_decoding.flash_decoding_stage2
    assert k.rms_norm is layer_ops.rms_norm and k.rotary_emb is layer_ops.rotary_emb
    assert k.silu_and_mul_inplace is layer_ops.silu_and_mul_inplace and k.ffn_block is layer_ops.ffn_block
    assert ns["longserve_c_scheduler"].minimize_prefill_iteration_time is scheduler.minimize_prefill_iteration_time
    assert ns["destindex_copy_kv"] is kv_ops.destindex_copy_kv and ns["copy_kv_index_to_req"] is kv_ops.copy_kv_index_to_req
    assert ns["pre_copy_and_register_kv"] is kv_ops.pre_copy_and_register_kv
    assert ns["destindex_copy_and_register_kv"] is kv_ops.destindex_copy_and_register_kv
    assert ns["decoding_stage_migration_sender_kernel"] is kv_ops.decoding_stage_migration_sender_kernel
    assert ns["decoding_stage_migration_receiver_kernel"] is kv_ops.decoding_stage_migration_receiver_kernel
    assert ns["init_req_to_token_indexes"] is kv_ops.init_req_to_token_indexes
    assert ns["longserve_token_decode_attention_flash_decoding"] is flash_decoding.longserve_token_decode_attention_flash_decoding
    assert ns["longserve_flash_decode_stage1"] is flash_decoding.longserve_flash_decode_stage1
    assert ns["longserve_flash_decode_stage2"] is flash_decoding.longserve_flash_decode_stage2
    assert ns["LongServeMemoryManager"] is mem_manager.LongServeMemoryManager and ns["LongServeReqManager"] is mem_manager.LongServeReqManager
    assert ns["prepare_prefill_inputs"] is pre_process.prepare_prefill_inputs and ns["prepare_decode_inputs"] is pre_process.prepare_decode_inputs
    assert "loongserve.models.llama.triton_kernel.ring_context_flashattention_nopad" in installed


def test_uninstall_restores_the_module_table():
    assert "longserve_cuda_kernels" not in sys.modules
    dropin.install()
    assert "longserve_cuda_kernels" in sys.modules
    dropin.uninstall()
    assert "longserve_cuda_kernels" not in sys.modules and "rnccl" not in sys.modules
    with pytest.raises(ImportError):
        importlib.import_module("longserve_cuda_kernels")


def test_unmodified_reference_modules_import_against_this_package():
    """With the reference checkout at hand (build container only), its layer-infer and model modules import unchanged
    and bind this package's kernels.  The checkout must be importable BEFORE install() so that its real parent packages
    are used."""
    import os
    from loongserve_b200.build import reference_dir
    ref = reference_dir()
    if ref is None or not os.path.isdir(os.path.join(ref, "loongserve", "models", "llama")):
        pytest.skip("reference checkout not present (set ESP_REFERENCE_DIR)")
    before = set(sys.modules)
    sys.path.insert(0, ref)
    try:
        dropin.install()
        li = importlib.import_module("loongserve.models.llama.layer_infer.longserve_transformer_layer_infer")
        lm = importlib.import_module("loongserve.models.llama.longserve_model")
        assert hasattr(li, "LongServeTransformerLayerInfer") and hasattr(lm, "LongServeLlamaModel")
        assert li.context_attention_fwd.__module__ == "loongserve_b200.context_attention"
        assert li.rnccl.RNCCLComm.__module__ == "loongserve_b200.rnccl"
        assert li.longserve_cuda_kernels.flash_decoding_stage1.__module__ == "loongserve_b200.flash_decoding"
        assert li.pre_copy_and_register_kv.__module__ == "loongserve_b200.kv_ops"
        assert lm.LongServeMemoryManager.__module__ == "loongserve_b200.mem_manager"
        assert lm.init_req_to_token_indexes.__module__ == "loongserve_b200.kv_ops"
    finally:
        dropin.uninstall()
        sys.path.remove(ref)
        for name in set(sys.modules) - before:
            if name.split(".")[0] in ("loongserve", "rnccl", "longserve_cuda_kernels", "longserve_c_scheduler"):
                sys.modules.pop(name, None)
