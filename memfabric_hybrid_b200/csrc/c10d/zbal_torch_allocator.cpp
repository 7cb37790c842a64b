// PyTorch allocator glue: the symmetric-heap allocator (SMA) as a CUDAPluggableAllocator WITH the
// capture hooks, so that CUDA graphs captured under it get private pools.
//
// torch.cuda.memory.CUDAPluggableAllocator (the Python class) can only set the malloc / free pair. The pool
// hooks (begin / end allocate-to-pool, release pool) and the reset hook exist on the C++ object only, so the
// allocator object is built here and handed to Python as a torch._C._cuda_CUDAAllocator, usable with
// torch.cuda.memory.change_current_allocator's C++ counterpart (install_global) or with torch.cuda.MemPool.
//
// Parity of role: the graph-capture private pools of app/zbal/src/csrc/sma and
// adaptor/pytorch_npu/zbal_pytorch_c10_dma.cpp of the reference.
#include <torch/extension.h>

#include <torch/csrc/cuda/CUDAPluggableAllocator.h>

#include <map>
#include <mutex>

#include "zbal_mem_allocator.h"

namespace zbal_c10d {
namespace {

using Filter = std::function<bool(cudaStream_t)>;
using PoolKey = std::pair<uint64_t, uint64_t>;

std::mutex g_mu;
std::map<PoolKey, Filter *> g_filters;  // alive from begin to end of routing
std::shared_ptr<c10::cuda::CUDACachingAllocator::CUDAAllocator> g_allocator;

bool FilterThunk(void *ctx, zbal_stream_t stream) { return (*static_cast<Filter *>(ctx))(static_cast<cudaStream_t>(stream)); }

std::shared_ptr<c10::cuda::CUDACachingAllocator::CUDAAllocator> Allocator()
{
    std::lock_guard<std::mutex> g(g_mu);
    if (g_allocator) return g_allocator;
    namespace P = torch::cuda::CUDAPluggableAllocator;
    auto base = P::createCustomAllocator(
        [](size_t n, int dev, cudaStream_t s) { return zbal_pluggable_malloc(n, dev, s); },
        [](void *p, size_t n, int dev, cudaStream_t s) { zbal_pluggable_free(p, n, dev, s); });
    auto *pa = dynamic_cast<P::CUDAPluggableAllocator *>(base.get());
    TORCH_CHECK(pa != nullptr, "zbal: createCustomAllocator did not return a CUDAPluggableAllocator");
    pa->set_reset_fn([]() { zbal_pluggable_empty_cache(false); });
    pa->set_begin_allocate_to_pool([](int, c10::cuda::MempoolId_t id, Filter filter) {
        auto *f = new Filter(std::move(filter));
        Filter *old = nullptr;
        {
            std::lock_guard<std::mutex> g2(g_mu);
            auto &slot = g_filters[{id.first, id.second}];
            old = slot;
            slot = f;
        }
        int32_t rc = zbal_sma_begin_pool(id.first, id.second, FilterThunk, f);
        delete old;
        TORCH_CHECK(rc == 0, "zbal_sma_begin_pool failed (", rc, ")");
    });
    pa->set_end_allocate_to_pool_fn([](int, c10::cuda::MempoolId_t id) {
        zbal_sma_end_pool(id.first, id.second);  // the allocator forgets the filter before it is deleted
        Filter *f = nullptr;
        {
            std::lock_guard<std::mutex> g2(g_mu);
            auto it = g_filters.find({id.first, id.second});
            if (it != g_filters.end()) {
                f = it->second;
                g_filters.erase(it);
            }
        }
        delete f;
    });
    pa->set_release_pool([](int, c10::cuda::MempoolId_t id) { zbal_sma_release_pool(id.first, id.second); });
    g_allocator = base;
    return g_allocator;
}

}  // namespace

void BindAllocator(py::module_ &m)
{
    m.def("allocator", &Allocator,
          "The symmetric-heap allocator as a torch._C._cuda_CUDAAllocator with the CUDA-graph pool hooks set "
          "(pass it to torch.cuda.MemPool, or call install_global_allocator()).");
    m.def(
        "install_global_allocator",
        []() { torch::cuda::CUDAPluggableAllocator::changeCurrentAllocator(Allocator()); },
        "Makes the symmetric-heap allocator the process-wide CUDA allocator. Only possible before the first CUDA "
        "allocation of the process.");
}

}  // namespace zbal_c10d
