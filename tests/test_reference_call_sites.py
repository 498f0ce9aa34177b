"""Every call the reference makes into the replaced functions binds to this package's signatures, and every attribute it
reads from the pool managers and the communicator exists here.  The call sites are taken from the reference's own source
files (parsed, not executed), so this runs only where the reference checkout is present."""
import ast
import inspect
import os

import pytest
import torch

from loongserve_b200 import dropin, mem_manager, rnccl
from loongserve_b200.build import reference_dir

REF = reference_dir() or ""
FILES = ["loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py", "loongserve/models/llama/longserve_model.py",
         "loongserve/longserve_server/router/manager.py", "loongserve/longserve_server/router/model_infer/model_rpc.py"]

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "loongserve", "models", "llama")),
                                reason="reference checkout not present (set ESP_REFERENCE_DIR)")


def _trees():
    for fn in FILES:
        with open(os.path.join(REF, fn)) as f:
            yield fn, ast.parse(f.read())


def _callee(f):
    if isinstance(f, ast.Name):
        return f.id
    if isinstance(f, ast.Attribute) and isinstance(f.value, ast.Name):
        return f.value.id + "." + f.attr
    return None


def test_every_reference_call_binds_to_our_signature():
    table = {}
    for path, mod in dropin.alias_table().items():
        for k, v in vars(mod).items():
            if callable(v) and not k.startswith("__"):
                table[k] = v
                table[path.split(".")[-1] + "." + k] = v
    for names in dropin.patch_table().values():
        table.update(names)
    seen = 0
    for fn, tree in _trees():
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and _callee(node.func) in table:
                target = table[_callee(node.func)]
                is_class = inspect.isclass(target)
                sig = inspect.signature(target.__init__ if is_class else target)
                args = [None] * (len(node.args) + (1 if is_class else 0))
                kwargs = {k.arg: None for k in node.keywords if k.arg}
                try:
                    sig.bind(*args, **kwargs)
                except TypeError as e:
                    raise AssertionError(f"{fn}:{node.lineno} {_callee(node.func)}: {e}") from None
                seen += 1
    assert seen >= 20           # the layer-infer, model, router and worker call sites


def test_every_attribute_the_reference_reads_from_managers_and_communicator_exists():
    mm = mem_manager.LongServeMemoryManager(8, torch.float16, 1, 8, 1, device="cpu")
    rm = mem_manager.LongServeReqManager(2, 4, mm)
    owners = {"mem_manager": mm, "req_manager": rm, "sp_comm": rnccl.RNCCLComm}
    used = {k: set() for k in owners}
    for fn, tree in list(_trees())[:2]:
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Attribute) and node.value.attr in owners:
                used[node.value.attr].add(node.attr)
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id in owners:
                used[node.value.id].add(node.attr)
    assert used["mem_manager"] and used["sp_comm"]
    for owner, attrs in used.items():
        for a in sorted(attrs):
            assert hasattr(owners[owner], a), f"the reference uses {owner}.{a}"
