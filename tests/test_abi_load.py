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
    assert capi.lib().kvmig_abi_version() == 2
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


def _handle_checksum(words):
    """The handle's last word: a hash over the 23 words before it (kvmig.cu: handle_checksum)."""
    mask = (1 << 64) - 1
    h = 0x9E3779B97F4A7C15
    for w in words[:23]:
        h ^= ((w & mask) + 0x9E3779B97F4A7C15 + ((h << 6) & mask) + (h >> 2)) & mask
    return h - (1 << 64) if h >= (1 << 63) else h


def test_a_handle_with_this_pid_but_another_process_number_is_not_local(built_libs):
    """Two workers in different pid namespaces can carry the same pid, so the pid alone must not make a
    handle "exported by this process" (such a handle's raw address is dereferenced): the per-process number
    drawn at start-up has to match as well.  Forged here without a device: well-formed words, this pid, a
    different number."""
    from distserve_b200 import capi

    magic = 0x4B564D4947303031
    words = [0] * capi.HANDLE_WORDS
    words[0] = magic
    words[10] = 8 * 2 * 2 * 4 * 8 * 2                     # pool bytes for the shape below
    words[11] = os.getpid()
    words[12] = 0x7F0000000000                            # "address" in the forging process
    words[14:20] = [8, 2, 2, 4, 8, 2]
    words[21] = 12345                                     # not this process's number
    words[23] = _handle_checksum(words)
    assert capi.handle_is_local(words) is False
    words[11] = os.getpid() + 1
    words[23] = _handle_checksum(words)
    assert capi.handle_is_local(words) is False
    words[23] ^= 1
    with pytest.raises(capi.KvmigError, match="checksum"):
        capi.handle_is_local(words)


@pytest.mark.gpu
def test_exported_handles_are_local_only_with_their_process_number(built_libs):
    from distserve_b200 import capi

    pool = torch.zeros(8, 2, 2, 4, 8, dtype=torch.float16, device="cuda")
    shape = capi.PoolShape.of(*pool.shape, 2)
    words = capi.get_ipc_mem_handle(pool.data_ptr(), shape)
    assert words[23] == _handle_checksum(words)           # the test's restatement of the checksum is the library's
    assert capi.handle_is_local(words) is True
    forged = list(words)
    forged[21] ^= 0x55
    forged[23] = _handle_checksum(forged)
    assert capi.handle_is_local(forged) is False
    # registering the forged handle takes the other-process route (CUDA IPC) instead of trusting the raw address:
    # either CUDA refuses to open a handle of the opening process itself, or the open shows in the counter
    capi.reset_registry()
    opened = capi.get_counter("mapped_peers")
    try:
        capi.register_ipc_mem_handle(forged, forged, 2, 2, [1, 0, 1, 0], [1, 0, 1, 0])
    except capi.KvmigError as e:
        assert e.code == capi.ECUDA and "cudaIpcOpenMemHandle" in str(e)
    else:
        assert capi.get_counter("mapped_peers") == opened + 1
    capi.reset_registry()
    capi.register_ipc_mem_handle(words, words, 2, 2, [1, 0, 1, 0], [1, 0, 1, 0])
    assert capi.get_counter("mapped_peers") <= opened + 1     # the genuine handle needed no IPC open
    capi.reset_registry()


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


def test_block_lists_are_packed_as_int64(built_libs):
    """The binding hands block lists to the C ABI as int64 arrays: values survive, an empty list still yields a
    valid pointer, numpy integers are accepted and non-integers refused."""
    import numpy as np

    from distserve_b200 import capi

    arr = capi.as_i64([5, 0, 2**40, -1])
    assert list(arr) == [5, 0, 2**40, -1] and len(arr) == 4
    assert len(capi.as_i64([])) == 1                      # never a zero-length ctypes array
    assert list(capi.as_i64((np.int64(7), np.int32(3)))) == [7, 3]
    with pytest.raises(TypeError):
        capi.as_i64([1.5])
    boxed = capi.I64List(range(10))
    assert len(boxed) == 10 and list(boxed.array) == list(range(10))
