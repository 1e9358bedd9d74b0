"""The shared libraries load on a machine without a GPU, export every symbol
the header declares, and refuse bad arguments before touching CUDA."""
import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "kvmig.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"KVMIG_API\s+[\w\s\*]+?\b(kvmig_\w+)\s*\(", text)))


def test_header_and_binding_agree(built_libs):
    from distserve_b200 import capi

    names = declared_symbols()
    assert len(names) >= 12
    assert sorted(capi.SIGNATURES) == names
    lib = ctypes.CDLL(str(built_libs[0]))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/kvmig.h but not exported"
    assert capi.lib().kvmig_abi_version() == 1
    m = re.search(r"#define KVMIG_HANDLE_WORDS (\d+)", HEADER.read_text())
    assert int(m.group(1)) == capi.HANDLE_WORDS


def test_only_the_c_abi_is_exported(built_libs):
    out = subprocess.run(["nm", "-D", "--defined-only", str(built_libs[0])], capture_output=True, text=True, check=True).stdout
    exported = [line.split()[-1] for line in out.splitlines() if " T " in line]
    assert sorted(exported) == declared_symbols()


def test_validation_happens_before_cuda(built_libs):
    from distserve_b200 import capi

    shape = capi.PoolShape.of(8, 2, 2, 4, 8, 2)
    with pytest.raises(capi.KvmigError) as e:
        capi.migrate_blocks(1, 1, [0, 1], 1, 1, 0, 0, [0], 0x1000, 0x2000, shape)
    assert e.value.code == capi.EINVAL and "2 entries" in str(e.value)
    with pytest.raises(capi.KvmigError) as e:
        capi.register_ipc_mem_handle([1, 2, 3], [1, 2, 3], 4, 4, [1, 0, 1, 0], [1, 0, 1, 0])
    assert e.value.code == capi.EINVAL and "24" in str(e.value)
    words = [0] * capi.HANDLE_WORDS
    with pytest.raises(capi.KvmigError, match="bad magic"):
        capi.register_ipc_mem_handle(words, words, 4, 4, [1, 0, 1, 0], [1, 0, 1, 0])
    with pytest.raises(capi.KvmigError) as e:
        capi.swap([0, 9], [0, 1], True, 0x1000, 0x2000, shape, 0x3000, 0x4000, 4)
    assert e.value.code == capi.EINVAL and "outside the host pool" in str(e.value)
    bad = capi.PoolShape.of(8, 0, 2, 4, 8, 2)
    with pytest.raises(capi.KvmigError, match="non-positive"):
        capi.swap([], [], True, 0x1000, 0x2000, bad, 0x3000, 0x4000, 4)
    with pytest.raises(capi.KvmigError, match="unknown option"):
        capi.set_option("no_such_option", 1)
    with pytest.raises(capi.KvmigError):
        capi.set_option("chunk_bytes", 100)      # not a multiple of 16
    assert capi.get_option("chunk_bytes") % 16 == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_compute_fails_loudly_without_a_gpu(built_libs):
    from distserve_b200 import capi

    shape = capi.PoolShape.of(8, 2, 2, 4, 8, 2)
    with pytest.raises(capi.KvmigError) as e:
        capi.migrate_blocks(1, 1, [0], 1, 1, 0, 0, [1], 0x1000, 0x2000, shape)
    assert e.value.code == capi.ECUDA
    with pytest.raises(capi.KvmigError) as e:
        capi.get_ipc_mem_handle(0x1000, shape)
    assert e.value.code == capi.ECUDA
    from distserve_b200.config import CacheConfig, KVModelConfig
    from distserve_b200.worker import KVWorker

    with pytest.raises(RuntimeError, match="CUDA device"):
        KVWorker(0, "decoding", KVModelConfig(2, 2, 8), CacheConfig(4, 8))


def test_shim_registers_the_reference_operator_names(built_libs):
    import distserve_b200

    distserve_b200.load_ops()
    schemas = {
        # operator -> argument types in call order (distserve/worker.py:133-134,239-246,256-267,303-311)
        "block_migration_ops::get_ipc_mem_handle": ["Tensor"],
        "block_migration_ops::register_ipc_mem_handle": ["List[int]", "List[int]", "int", "int", "List[int]", "List[int]"],
        "block_migration_ops::migrate_blocks": ["int", "int", "List[int]", "int", "int", "int", "int", "List[int]", "Tensor", "Tensor"],
        "swapping_ops::swap": ["List[int]", "List[int]", "bool", "Tensor", "Tensor", "Tensor", "Tensor"],
    }
    for qualified, expected in schemas.items():
        ns, name = qualified.split("::")
        op = getattr(getattr(torch.ops, ns), name)
        assert [str(a.type) for a in op.default._schema.arguments] == expected, qualified
    # host tensors are rejected by the shim itself, before the C ABI is reached
    k = torch.zeros(4, 2, 2, 4, 8, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        torch.ops.block_migration_ops.migrate_blocks(1, 1, [0], 1, 1, 0, 0, [1], k, k.clone())
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        torch.ops.block_migration_ops.get_ipc_mem_handle(k)
    with pytest.raises(RuntimeError, match="24"):
        torch.ops.block_migration_ops.register_ipc_mem_handle([1], [2], 4, 4, [1, 0, 1, 0], [1, 0, 1, 0])


REFERENCE = Path(os.environ.get("DISTSERVE_REFERENCE_DIR", ROOT.parent / "reference"))   # a checkout beside this repo


@pytest.mark.skipif(not (REFERENCE / "distserve").is_dir(), reason="reference checkout not present")
def test_unmodified_reference_package_loads_our_library(built_libs):
    """distserve/__init__.py loads whatever SWIFT_TRANSFORMER_LIB_PATH names;
    with the shim there, the reference's worker module finds all four operators."""
    code = f"""
import sys, types
ray = types.ModuleType('ray'); ray.remote = lambda *a, **k: (lambda cls: cls); ray.get_gpu_ids = lambda: [0]
for n in ('ray.util', 'ray.util.placement_group', 'ray.util.scheduling_strategies'):
    sys.modules[n] = types.ModuleType(n)
sys.modules['ray.util.placement_group'].PlacementGroup = object
sys.modules['ray.util.scheduling_strategies'].PlacementGroupSchedulingStrategy = object
ray.util = sys.modules['ray.util']; sys.modules['ray'] = ray
sys.path.insert(0, {str(REFERENCE)!r})
import warnings; warnings.simplefilter('ignore')
import torch, distserve, distserve.worker, distserve.block_manager
for ns, op in (('block_migration_ops', 'get_ipc_mem_handle'), ('block_migration_ops', 'register_ipc_mem_handle'),
               ('block_migration_ops', 'migrate_blocks'), ('swapping_ops', 'swap')):
    getattr(getattr(torch.ops, ns), op)
print('LOADED', distserve.LIB_PATH)
"""
    env = dict(os.environ, SWIFT_TRANSFORMER_LIB_PATH=str(built_libs[1]))
    proc = subprocess.run([sys.executable, "-W", "ignore", "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert f"LOADED {built_libs[1]}" in proc.stdout
