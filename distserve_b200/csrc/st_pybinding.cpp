// Operator shim: registers the operator names DistServe's Python layer calls
// (torch.ops.block_migration_ops.* and torch.ops.swapping_ops.swap) and
// forwards them to the C ABI of libkvmig.so.  Built as libst_pybinding.so so
// that pointing SWIFT_TRANSFORMER_LIB_PATH at it makes distserve/__init__.py:4-16
// load this library in place of SwiftTransformer's.
//
// The shim only unpacks tensors (address, sizes, element size, device), picks
// up the ambient CUDA stream, and turns a non-zero status into a C++ exception
// (a Python RuntimeError), which is the reference's error convention: nothing
// catches it and the server exits (distserve/api_server/distserve_api_server.py:148-155).
#include <torch/library.h>
#include <ATen/core/Tensor.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/util/ArrayRef.h>

#include <vector>

#include "../../include/kvmig.h"

namespace {

void check(int rc, const char* op) {
    TORCH_CHECK(rc == 0, op, ": ", kvmig_last_error(), " (kvmig status ", rc, ")");
}

kvmig_pool_shape pool_shape(const at::Tensor& t, const char* name) {
    TORCH_CHECK(t.dim() == 5, name, " must have 5 dimensions [num_blocks, num_layers, num_heads, block_size, head_dim], got ",
                t.dim());
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    kvmig_pool_shape s;
    s.num_blocks = t.size(0);
    s.num_layers = t.size(1);
    s.num_heads = t.size(2);
    s.block_size = t.size(3);
    s.head_dim = t.size(4);
    s.elem_size = static_cast<int64_t>(t.element_size());
    return s;
}

void check_pair(const at::Tensor& k, const at::Tensor& v, const char* kn, const char* vn) {
    TORCH_CHECK(k.sizes() == v.sizes(), kn, " and ", vn, " differ in shape");
    TORCH_CHECK(k.scalar_type() == v.scalar_type(), kn, " and ", vn, " differ in dtype");
    TORCH_CHECK(k.device() == v.device(), kn, " and ", vn, " are on different devices");
}

// block_migration_ops::get_ipc_mem_handle(Tensor) -> int[]     (distserve/worker.py:133-134)
std::vector<int64_t> get_ipc_mem_handle(const at::Tensor& pool) {
    TORCH_CHECK(pool.is_cuda(), "get_ipc_mem_handle: the pool must be a CUDA tensor");
    kvmig_pool_shape s = pool_shape(pool, "pool");
    c10::cuda::CUDAGuard guard(pool.device());
    std::vector<int64_t> words(KVMIG_HANDLE_WORDS);
    check(kvmig_get_ipc_mem_handle(pool.data_ptr(), &s, words.data()), "get_ipc_mem_handle");
    return words;
}

// block_migration_ops::register_ipc_mem_handle(...)            (distserve/worker.py:239-246)
bool register_ipc_mem_handle(c10::IntArrayRef k_handle, c10::IntArrayRef v_handle, int64_t num_layers,
                             int64_t num_heads, c10::IntArrayRef context_parallel_config,
                             c10::IntArrayRef decoding_parallel_config) {
    TORCH_CHECK(context_parallel_config.size() == 4 && decoding_parallel_config.size() == 4,
                "register_ipc_mem_handle: parallel configs must be [tp_size, tp_rank, pp_size, pp_rank]");
    check(kvmig_register_ipc_mem_handle(k_handle.data(), static_cast<int64_t>(k_handle.size()), v_handle.data(),
                                        static_cast<int64_t>(v_handle.size()), num_layers, num_heads,
                                        context_parallel_config.data(), decoding_parallel_config.data()),
          "register_ipc_mem_handle");
    return true;
}

// block_migration_ops::migrate_blocks(...)                     (distserve/worker.py:256-267)
// The block lists are views of the caller's arguments (no copy); the tensors are taken by reference.
void migrate_blocks(int64_t context_pp_size, int64_t context_tp_size, c10::IntArrayRef context_block_indexes,
                    int64_t decoding_pp_size, int64_t decoding_tp_size, int64_t decoding_pp_rank,
                    int64_t decoding_tp_rank, c10::IntArrayRef decoding_block_indexes, const at::Tensor& k_cache,
                    const at::Tensor& v_cache) {
    TORCH_CHECK(k_cache.is_cuda() && v_cache.is_cuda(), "migrate_blocks: k_cache and v_cache must be CUDA tensors");
    check_pair(k_cache, v_cache, "k_cache", "v_cache");
    kvmig_pool_shape s = pool_shape(k_cache, "k_cache");
    TORCH_CHECK(v_cache.is_contiguous(), "v_cache must be contiguous");
    // Switch devices only when the pool is not on the current one (a worker process owns one GPU).
    c10::cuda::OptionalCUDAGuard guard;
    if (c10::cuda::current_device() != k_cache.device().index()) guard.set_device(k_cache.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(k_cache.device().index()).stream();
    check(kvmig_migrate_blocks(context_pp_size, context_tp_size, context_block_indexes.data(),
                               static_cast<int64_t>(context_block_indexes.size()), decoding_pp_size, decoding_tp_size,
                               decoding_pp_rank, decoding_tp_rank, decoding_block_indexes.data(),
                               static_cast<int64_t>(decoding_block_indexes.size()), k_cache.data_ptr(), v_cache.data_ptr(),
                               &s, stream),
          "migrate_blocks");
}

// swapping_ops::swap(...)                                      (distserve/worker.py:303-311)
void swap(c10::IntArrayRef source_block_ids, c10::IntArrayRef target_block_ids, bool is_swap_in,
          const at::Tensor& k_cache, const at::Tensor& v_cache, const at::Tensor& k_swap, const at::Tensor& v_swap) {
    TORCH_CHECK(k_cache.is_cuda() && v_cache.is_cuda(), "swap: k_cache and v_cache must be CUDA tensors");
    TORCH_CHECK(k_swap.is_cpu() && v_swap.is_cpu(), "swap: k_swap and v_swap must be host tensors");
    check_pair(k_cache, v_cache, "k_cache", "v_cache");
    check_pair(k_swap, v_swap, "k_swap", "v_swap");
    kvmig_pool_shape s = pool_shape(k_cache, "k_cache");
    (void)pool_shape(v_cache, "v_cache");
    kvmig_pool_shape hs = pool_shape(k_swap, "k_swap");
    (void)pool_shape(v_swap, "v_swap");
    TORCH_CHECK(k_swap.scalar_type() == k_cache.scalar_type(), "swap: host and GPU pools differ in dtype");
    TORCH_CHECK(hs.num_layers == s.num_layers && hs.num_heads == s.num_heads && hs.block_size == s.block_size &&
                    hs.head_dim == s.head_dim,
                "swap: host and GPU pools differ in per-block shape");
    c10::cuda::CUDAGuard guard(k_cache.device());
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(k_cache.device().index()).stream();
    check(kvmig_swap(source_block_ids.data(), static_cast<int64_t>(source_block_ids.size()), target_block_ids.data(),
                     static_cast<int64_t>(target_block_ids.size()), is_swap_in ? 1 : 0, k_cache.data_ptr(),
                     v_cache.data_ptr(), &s, k_swap.data_ptr(), v_swap.data_ptr(), hs.num_blocks, stream),
          "swap");
}

}  // namespace

TORCH_LIBRARY(block_migration_ops, m) {
    m.def("get_ipc_mem_handle(Tensor pool) -> int[]", &get_ipc_mem_handle);
    m.def("register_ipc_mem_handle(int[] k_handle, int[] v_handle, int num_layers, int num_heads, "
          "int[] context_parallel_config, int[] decoding_parallel_config) -> bool",
          &register_ipc_mem_handle);
    m.def("migrate_blocks(int context_pp_size, int context_tp_size, int[] context_block_indexes, "
          "int decoding_pp_size, int decoding_tp_size, int decoding_pp_rank, int decoding_tp_rank, "
          "int[] decoding_block_indexes, Tensor k_cache, Tensor v_cache) -> ()",
          &migrate_blocks);
}

TORCH_LIBRARY(swapping_ops, m) {
    m.def("swap(int[] source_block_ids, int[] target_block_ids, bool is_swap_in, Tensor k_cache, Tensor v_cache, "
          "Tensor k_swap, Tensor v_swap) -> ()",
          &swap);
}
