"""B200-native (sm_100a) elastic-sequence-parallel attention hot path.

The modules mirror the call surface of the reference's model layer for this path:

  context_attention   context_attention_fwd                      (ring-prefill attention step)
  flash_decoding      flash_decoding_stage1 / _stage2 and the    (distributed flash-decoding)
                      longserve_flash_decode_* wrappers
  kv_ops              destindex_copy_kv, pre_copy_and_register_kv, destindex_copy_and_register_kv,
                      copy_kv_index_to_req, init_req_to_token_indexes,
                      decoding_stage_migration_{sender,receiver}_kernel
  mem_manager         LongServeMemoryManager, LongServeReqManager  (token-indexed KV pool)
  rnccl               get_nccl_unique_id, RNCCLComm               (raw NCCL point-to-point)
  ring                ring prefill loop and multi-master decode orchestration

All compute goes through the C ABI in include/esp_attention.h; there is no CPU or PyTorch fallback.
"""
from . import _lib  # noqa: F401

__all__ = ["context_attention", "flash_decoding", "kv_ops", "mem_manager", "rnccl", "ring"]
