// torch.distributed backend "zbal" as a native c10d::Backend.
//
// Collectives of contiguous CUDA tensors run as zbal kernels over NVLink peer memory (the zbal C API of
// libmf_smem.so, which this module links); everything else goes to a fallback backend that the Python side
// builds on demand (NCCL for CUDA tensors, gloo for host tensors).
//
// Parity: app/zbal/src/csrc/adaptor/pytorch_npu/zbal_pytorch_process_group.{h,cpp} of the reference
// (method set h:130-166, stream discipline cpp:312-367, lazy pair communicators h:164-166). The stream
// discipline is the same: one side stream per group; the operation first waits on an event recorded on the
// caller's stream, runs, and records an end event into the returned Work; Work::wait() makes the CALLER's
// stream wait on that event and the host does not block. ZBAL_OP_DEFAULT_STREAM=1 runs operations on the
// caller's stream directly.
#include <torch/extension.h>

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/chrono.h>
#include <pybind11/functional.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <sstream>
#include <tuple>

#include "zbal.h"
#include "zbal_bootstrap.h"
#include "zbal_operations.h"

namespace zbal_c10d {

using c10d::Work;
using TensorList = std::vector<at::Tensor>;

static int DtypeOf(at::ScalarType t)
{
    switch (t) {
        case at::kChar: return ZBAL_DT_INT8;
        case at::kShort: return ZBAL_DT_INT16;
        case at::kInt: return ZBAL_DT_INT32;
        case at::kLong: return ZBAL_DT_INT64;
        case at::kDouble: return ZBAL_DT_FP64;
        case at::kHalf: return ZBAL_DT_FP16;
        case at::kFloat: return ZBAL_DT_FP32;
        case at::kBFloat16: return ZBAL_DT_BF16;
        case at::kByte:
        case at::kBool:
        case at::kFloat8_e4m3fn:
        case at::kFloat8_e5m2: return ZBAL_DT_UINT8;
        default: return -1;
    }
}

static bool Reducible(at::ScalarType t) { return t == at::kBFloat16 || t == at::kHalf || t == at::kFloat || t == at::kInt; }

static int ReduceOpOf(const c10d::ReduceOp &op, bool &avg)
{
    avg = false;
    switch (op.op_) {
        case c10d::ReduceOp::SUM: return ZBAL_REDUCE_SUM;
        case c10d::ReduceOp::AVG: avg = true; return ZBAL_REDUCE_SUM;
        case c10d::ReduceOp::PRODUCT: return ZBAL_REDUCE_PROD;
        case c10d::ReduceOp::MIN: return ZBAL_REDUCE_MIN;
        case c10d::ReduceOp::MAX: return ZBAL_REDUCE_MAX;
        default: return -1;
    }
}

static void Check(int32_t rc, const char *what)
{
    if (rc != 0) {
        const char *msg = zbal_get_last_error_msg();
        TORCH_CHECK(false, what, " failed (", rc, "): ", msg ? msg : "");
    }
}

static std::string EnvOr(const char *name, const char *dflt)
{
    const char *v = std::getenv(name);
    return (v != nullptr && *v != 0) ? std::string(v) : std::string(dflt);
}

// ---------------------------------------------------------------------------------------------------
class WorkZBAL : public Work {
public:
    WorkZBAL(int rank, c10d::OpType op, TensorList outputs, std::shared_ptr<at::cuda::CUDAEvent> done, c10::DeviceIndex dev,
             TensorList keep)
        : Work(rank, op), outputs_(std::move(outputs)), done_(std::move(done)), dev_(dev), keep_(std::move(keep))
    {
    }

    bool isCompleted() override { return !done_ || done_->query(); }
    bool isSuccess() const override { return true; }

    // The caller's stream waits; the host goes on (cpp:352-367 of the reference do the same with NPU events).
    bool wait(std::chrono::milliseconds /*timeout*/ = kNoTimeout) override
    {
        if (done_) done_->block(c10::cuda::getCurrentCUDAStream(dev_));
        return true;
    }
    void synchronize() override { wait(); }
    void blockCurrentStream() override { wait(); }
    void hostSynchronize()
    {
        if (done_) done_->synchronize();
    }
    std::vector<at::Tensor> result() override { return outputs_; }

    c10::intrusive_ptr<c10::ivalue::Future> getFuture() override
    {
        if (!future_) {
            // Completed at once, as in the reference (cpp:352-355): consumers order themselves by wait().
            // The future is told which device its tensors live on: it records an event on the current stream when it
            // is completed (after that stream was made to wait for the operation) and its consumers wait on that event.
            future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                               std::vector<c10::Device>{c10::Device(c10::kCUDA, dev_)});
            wait();
            future_->markCompleted(c10::IValue(outputs_));
        }
        return future_;
    }

private:
    TensorList outputs_;
    std::shared_ptr<at::cuda::CUDAEvent> done_;
    c10::DeviceIndex dev_;
    TensorList keep_;
    c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// ---------------------------------------------------------------------------------------------------
class ProcessGroupZBAL : public c10d::Backend {
public:
    using Factory = std::function<c10::intrusive_ptr<c10d::Backend>(bool)>;

    ProcessGroupZBAL(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, std::vector<int64_t> ranks,
                     std::chrono::milliseconds timeout)
        : Backend(rank, size), store_(store), ranks_(std::move(ranks)), timeout_(timeout)
    {
        if (ranks_.empty())
            for (int i = 0; i < size; i++) ranks_.push_back(i);
        TORCH_CHECK((int)ranks_.size() == size, "zbal: ", ranks_.size(), " global ranks for a group of ", size);
        strided_ = true;
        if (size > 1) {
            int64_t step = ranks_[1] - ranks_[0];
            strided_ = step > 0;
            for (int i = 0; strided_ && i + 1 < size; i++) strided_ = ranks_[i + 1] - ranks_[i] == step;
        }
        std::stringstream forced(EnvOr("ZBAL_NCCL_OP", EnvOr("ZBAL_HCCL_OP", "").c_str()));  // the second name is the reference's
        for (std::string item; std::getline(forced, item, ',');) {
            size_t a = item.find_first_not_of(' '), b = item.find_last_not_of(' ');
            if (a != std::string::npos) forced_.insert(item.substr(a, b - a + 1));
        }
        ownStream_ = EnvOr("ZBAL_OP_DEFAULT_STREAM", EnvOr("ZBAL_OP_DEFUALT_STREAM", "0").c_str()) != "1";
        {
            std::lock_guard<std::mutex> g(Mu());
            Live().insert(this);
        }
        if (zbal_is_bootstrapped() && strided_) Communicator();
    }

    ~ProcessGroupZBAL() override
    {
        {
            std::lock_guard<std::mutex> g(Mu());
            Live().erase(this);
        }
        DropFactory();
    }

    const std::string getBackendName() const override { return "zbal"; }
    void setSequenceNumberForGroup() override {}
    uint64_t getSequenceNumberForGroup() override { return seq_; }

    // Called by the Python side of zbal_uninit(): communicator handles die with the bootstrap.
    static void ForgetAll()
    {
        std::lock_guard<std::mutex> g(Mu());
        for (auto *pg : Live()) {
            pg->comm_ = nullptr;
            pg->pairs_.clear();
        }
        Counters().clear();
    }

    void SetFallbackFactory(py::function f)
    {
        DropFactory();
        factory_ = new py::function(std::move(f));
    }

    void shutdown() override
    {
        nccl_.reset();
        gloo_.reset();
        DropFactory();
    }

    std::string CommName()
    {
        zbal_comm_property_t p{};
        Check(zbal_comm_get_property(Communicator(), &p), "zbal_comm_get_property");
        return std::string(p.name);
    }
    uint64_t CommHandle() { return reinterpret_cast<uint64_t>(Communicator()); }
    bool Strided() const { return strided_; }

    std::vector<uint32_t> DeviceStatus()
    {
        uint32_t st[4] = {0, 0, 0, 0};
        Check(zbal_comm_get_device_status(Communicator(), st), "zbal_comm_get_device_status");
        return {st[0], st[1], st[2], st[3]};
    }

    // ---------------------------------------------------------------- collectives
    c10::intrusive_ptr<Work> allreduce(TensorList &tensors, const c10d::AllreduceOptions &opts) override
    {
        bool avg = false;
        int op = ReduceOpOf(opts.reduceOp, avg);
        if (tensors.size() != 1 || op < 0 || !Reducible(tensors[0].scalar_type()) || !UseZbal("allreduce", tensors))
            return Fallback(tensors)->allreduce(tensors, opts);
        at::Tensor t = tensors[0];
        int dt = DtypeOf(t.scalar_type());
        float scale = avg ? 1.0f / (float)getSize() : 1.0f;
        zbal_comm_t comm = Communicator();
        return Run(c10d::OpType::ALLREDUCE, {t}, tensors, [=](zbal_stream_t s) {
            Check(zbal_all_reduce_scaled(t.data_ptr(), t.data_ptr(), (size_t)t.numel(), (zbal_datatype_t)dt, (zbal_datatype_t)dt,
                                         (zbal_reduce_op_t)op, scale, comm, s),
                  "zbal_all_reduce");
        });
    }

    c10::intrusive_ptr<Work> allreduce_coalesced(TensorList &tensors, const c10d::AllreduceCoalescedOptions &opts) override
    {
        return Fallback(tensors)->allreduce_coalesced(tensors, opts);
    }

    c10::intrusive_ptr<Work> reduce(TensorList &tensors, const c10d::ReduceOptions &opts) override
    {
        return Fallback(tensors)->reduce(tensors, opts);
    }

    c10::intrusive_ptr<Work> broadcast(TensorList &tensors, const c10d::BroadcastOptions &opts) override
    {
        if (tensors.size() != 1 || DtypeOf(tensors[0].scalar_type()) < 0 || !UseZbal("broadcast", tensors) || OddBytes(tensors[0]))
            return Fallback(tensors)->broadcast(tensors, opts);
        at::Tensor t = tensors[0];
        int dt = DtypeOf(t.scalar_type());
        auto root = (uint16_t)opts.rootRank;
        zbal_comm_t comm = Communicator();
        return Run(c10d::OpType::BROADCAST, {t}, tensors, [=](zbal_stream_t s) {
            Check(zbal_broadcast(t.data_ptr(), (uint64_t)t.numel(), (zbal_datatype_t)dt, root, comm, s), "zbal_broadcast");
        });
    }

    c10::intrusive_ptr<Work> _allgather_base(at::Tensor &output, at::Tensor &input, const c10d::AllgatherOptions &opts) override
    {
        TensorList both{output, input};
        if (DtypeOf(input.scalar_type()) < 0 || !UseZbal("_allgather_base", both) || OddBytes(input) ||
            output.numel() != input.numel() * getSize())
            return Fallback(both)->_allgather_base(output, input, opts);
        int dt = DtypeOf(input.scalar_type());
        zbal_comm_t comm = Communicator();
        at::Tensor in = input, out = output;
        return Run(c10d::OpType::_ALLGATHER_BASE, both, {output}, [=](zbal_stream_t s) {
            Check(zbal_all_gather(in.data_ptr(), out.data_ptr(), (size_t)in.numel(), (zbal_datatype_t)dt, comm, s), "zbal_all_gather");
        });
    }

    c10::intrusive_ptr<Work> allgather(std::vector<TensorList> &outputs, TensorList &inputs, const c10d::AllgatherOptions &opts) override
    {
        bool ok = inputs.size() == 1 && outputs.size() == 1 && DtypeOf(inputs[0].scalar_type()) >= 0 && UseZbal("allgather", inputs) &&
                  !OddBytes(inputs[0]) && (int)outputs[0].size() == getSize();
        for (size_t i = 0; ok && i < outputs[0].size(); i++)
            ok = outputs[0][i].numel() == inputs[0].numel() && outputs[0][i].is_cuda();
        if (!ok) return Fallback(inputs)->allgather(outputs, inputs, opts);
        at::Tensor in = inputs[0];
        TensorList outs = outputs[0];
        int dt = DtypeOf(in.scalar_type());
        at::Tensor flat = at::empty({(int64_t)getSize(), in.numel()}, in.options());
        zbal_comm_t comm = Communicator();
        TensorList touched{in, flat};
        touched.insert(touched.end(), outs.begin(), outs.end());
        return Run(c10d::OpType::ALLGATHER, touched, outs, [=](zbal_stream_t s) {
            Check(zbal_all_gather(in.data_ptr(), flat.data_ptr(), (size_t)in.numel(), (zbal_datatype_t)dt, comm, s), "zbal_all_gather");
            for (size_t r = 0; r < outs.size(); r++) outs[r].copy_(flat[r].view_as(outs[r]), true);
        });
    }

    c10::intrusive_ptr<Work> allgather_into_tensor_coalesced(TensorList &outputs, TensorList &inputs, const c10d::AllgatherOptions &opts) override
    {
        return Fallback(inputs)->allgather_into_tensor_coalesced(outputs, inputs, opts);
    }

    c10::intrusive_ptr<Work> gather(std::vector<TensorList> &outputs, TensorList &inputs, const c10d::GatherOptions &opts) override
    {
        if (inputs.size() != 1 || DtypeOf(inputs[0].scalar_type()) < 0 || !UseZbal("gather", inputs) || OddBytes(inputs[0]))
            return Fallback(inputs)->gather(outputs, inputs, opts);
        at::Tensor in = inputs[0];
        int dt = DtypeOf(in.scalar_type());
        auto root = (uint16_t)opts.rootRank;
        TensorList outs;
        if (getRank() == (int)opts.rootRank && !outputs.empty()) outs = outputs[0];
        at::Tensor flat = at::empty({(int64_t)getSize(), in.numel()}, in.options());
        zbal_comm_t comm = Communicator();
        TensorList touched{in, flat};
        touched.insert(touched.end(), outs.begin(), outs.end());
        return Run(c10d::OpType::GATHER, touched, outs, [=](zbal_stream_t s) {
            Check(zbal_gather(in.data_ptr(), flat.data_ptr(), (uint64_t)in.numel(), (zbal_datatype_t)dt, root, comm, s), "zbal_gather");
            for (size_t r = 0; r < outs.size(); r++) outs[r].copy_(flat[r].view_as(outs[r]), true);
        });
    }

    c10::intrusive_ptr<Work> scatter(TensorList &outputs, std::vector<TensorList> &inputs, const c10d::ScatterOptions &opts) override
    {
        if (outputs.size() != 1 || DtypeOf(outputs[0].scalar_type()) < 0 || !UseZbal("scatter", outputs) || OddBytes(outputs[0]))
            return Fallback(outputs)->scatter(outputs, inputs, opts);
        at::Tensor out = outputs[0];
        int dt = DtypeOf(out.scalar_type());
        auto root = (uint16_t)opts.rootRank;
        at::Tensor src;
        TensorList touched{out};
        if (getRank() == (int)opts.rootRank) {
            TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == getSize(), "zbal scatter: the root passes one tensor per rank");
            TensorList rows;
            for (auto &p : inputs[0]) rows.push_back(p.reshape({-1}));
            src = at::stack(rows).contiguous();
            touched.push_back(src);
        }
        zbal_comm_t comm = Communicator();
        return Run(c10d::OpType::SCATTER, touched, outputs, [=](zbal_stream_t s) {
            Check(zbal_scatter(src.defined() ? src.data_ptr() : nullptr, out.data_ptr(), (uint64_t)out.numel(), (zbal_datatype_t)dt, root,
                               comm, s),
                  "zbal_scatter");
        });
    }

    c10::intrusive_ptr<Work> _reduce_scatter_base(at::Tensor &output, at::Tensor &input, const c10d::ReduceScatterOptions &opts) override
    {
        bool avg = false;
        int op = ReduceOpOf(opts.reduceOp, avg);
        TensorList both{output, input};
        if (op < 0 || avg || !Reducible(input.scalar_type()) || !UseZbal("_reduce_scatter_base", both) ||
            input.numel() != output.numel() * getSize())
            return Fallback(both)->_reduce_scatter_base(output, input, opts);
        int dt = DtypeOf(input.scalar_type());
        zbal_comm_t comm = Communicator();
        at::Tensor in = input, out = output;
        return Run(c10d::OpType::_REDUCE_SCATTER_BASE, both, {output}, [=](zbal_stream_t s) {
            Check(zbal_reduce_scatter(in.data_ptr(), out.data_ptr(), (size_t)out.numel(), (zbal_datatype_t)dt, (zbal_reduce_op_t)op, comm, s),
                  "zbal_reduce_scatter");
        });
    }

    c10::intrusive_ptr<Work> reduce_scatter(TensorList &outputs, std::vector<TensorList> &inputs, const c10d::ReduceScatterOptions &opts) override
    {
        bool avg = false;
        int op = ReduceOpOf(opts.reduceOp, avg);
        bool ok = outputs.size() == 1 && inputs.size() == 1 && op >= 0 && !avg && Reducible(outputs[0].scalar_type()) &&
                  UseZbal("reduce_scatter", outputs) && (int)inputs[0].size() == getSize();
        for (size_t i = 0; ok && i < inputs[0].size(); i++) ok = inputs[0][i].numel() == outputs[0].numel() && inputs[0][i].is_cuda();
        if (!ok) return Fallback(outputs)->reduce_scatter(outputs, inputs, opts);
        at::Tensor out = outputs[0];
        int dt = DtypeOf(out.scalar_type());
        TensorList rows;
        for (auto &p : inputs[0]) rows.push_back(p.reshape({-1}));
        at::Tensor flat = at::stack(rows).contiguous();
        zbal_comm_t comm = Communicator();
        return Run(c10d::OpType::REDUCE_SCATTER, {flat, out}, outputs, [=](zbal_stream_t s) {
            Check(zbal_reduce_scatter(flat.data_ptr(), out.data_ptr(), (size_t)out.numel(), (zbal_datatype_t)dt, (zbal_reduce_op_t)op, comm, s),
                  "zbal_reduce_scatter");
        });
    }

    c10::intrusive_ptr<Work> reduce_scatter_tensor_coalesced(TensorList &outputs, TensorList &inputs,
                                                             const c10d::ReduceScatterOptions &opts) override
    {
        return Fallback(inputs)->reduce_scatter_tensor_coalesced(outputs, inputs, opts);
    }

    c10::intrusive_ptr<Work> alltoall(TensorList &outputs, TensorList &inputs, const c10d::AllToAllOptions &opts) override
    {
        return Fallback(inputs)->alltoall(outputs, inputs, opts);
    }

    c10::intrusive_ptr<Work> alltoall_base(at::Tensor &output, at::Tensor &input, std::vector<int64_t> &outSplits,
                                           std::vector<int64_t> &inSplits, const c10d::AllToAllOptions &opts) override
    {
        TensorList both{output, input};
        const int n = getSize();
        // the pieces land in the receiver's staging area: the larger of the two buffers sizes the call
        const uint64_t es = input.element_size(), nbytes = (uint64_t)std::max(input.numel(), output.numel()) * es;
        bool ok = DtypeOf(input.scalar_type()) >= 0 && UseZbal("alltoall_base", both) && nbytes % 2 == 0 && input.dim() >= 1 &&
                  output.dim() >= 1 && (inSplits.empty() || (int)inSplits.size() == n) && (outSplits.empty() || (int)outSplits.size() == n);
        if (ok) ok = nbytes + 4096 <= StageBytes();
        if (!ok) return Fallback(both)->alltoall_base(output, input, outSplits, inSplits, opts);
        const uint64_t rowIn = input.dim() > 1 ? (uint64_t)input[0].numel() : 1, rowOut = output.dim() > 1 ? (uint64_t)output[0].numel() : 1;
        at::Tensor meta = at::empty({n, 4}, at::TensorOptions().dtype(at::kLong).pinned_memory(true));
        auto *m = meta.data_ptr<int64_t>();
        uint64_t so = 0, ro = 0;
        for (int p = 0; p < n; p++) {
            uint64_t ni = inSplits.empty() ? (uint64_t)input.size(0) / n : (uint64_t)inSplits[p];
            uint64_t no = outSplits.empty() ? (uint64_t)output.size(0) / n : (uint64_t)outSplits[p];
            m[p * 4 + 0] = (int64_t)(so * rowIn * es);
            m[p * 4 + 1] = (int64_t)(ni * rowIn * es);
            m[p * 4 + 2] = (int64_t)(ro * rowOut * es);
            m[p * 4 + 3] = (int64_t)(no * rowOut * es);
            so += ni;
            ro += no;
        }
        at::Tensor devMeta = at::empty({n, 4}, input.options().dtype(at::kLong));
        zbal_comm_t comm = Communicator();
        at::Tensor in = input, out = output;
        return Run(c10d::OpType::ALLTOALL_BASE, {in, out, devMeta}, {output}, [=](zbal_stream_t s) {
            devMeta.copy_(meta, true);
            Check(zbal_all_to_all_v(in.data_ptr(), out.data_ptr(), (const uint64_t *)devMeta.data_ptr(), nbytes, comm, s), "zbal_all_to_all_v");
        });
    }

    c10::intrusive_ptr<Work> barrier(const c10d::BarrierOptions &opts) override
    {
        if (forced_.count("barrier") || !strided_ || !CudaReady()) return Fallback(CudaReady())->barrier(opts);
        zbal_comm_t comm = Communicator();
        auto work = Run(c10d::OpType::BARRIER, {}, {}, [=](zbal_stream_t s) { Check(zbal_barrier(comm, s), "zbal_barrier"); });
        static_cast<WorkZBAL *>(work.get())->hostSynchronize();  // a barrier returns when every rank has arrived
        return work;
    }

    c10::intrusive_ptr<Work> send(TensorList &tensors, int dst, int tag) override
    {
        if (tensors.size() != 1 || DtypeOf(tensors[0].scalar_type()) < 0 || !UseZbal("send", tensors))
            return Fallback(tensors)->send(tensors, dst, tag);
        at::Tensor t = tensors[0];
        int dt = DtypeOf(t.scalar_type());
        auto [comm, peer] = PairComm(dst);
        return Run(c10d::OpType::SEND, {t}, tensors, [=, comm = comm, peer = peer](zbal_stream_t s) {
            Check(zbal_send(t.data_ptr(), (size_t)t.numel(), (zbal_datatype_t)dt, peer, comm, s), "zbal_send");
        });
    }

    c10::intrusive_ptr<Work> recv(TensorList &tensors, int src, int tag) override
    {
        if (tensors.size() != 1 || DtypeOf(tensors[0].scalar_type()) < 0 || !UseZbal("recv", tensors))
            return Fallback(tensors)->recv(tensors, src, tag);
        at::Tensor t = tensors[0];
        int dt = DtypeOf(t.scalar_type());
        auto [comm, peer] = PairComm(src);
        return Run(c10d::OpType::RECV, {t}, tensors, [=, comm = comm, peer = peer](zbal_stream_t s) {
            Check(zbal_recv(t.data_ptr(), (size_t)t.numel(), (zbal_datatype_t)dt, peer, comm, s), "zbal_recv");
        });
    }

    c10::intrusive_ptr<Work> recvAnysource(TensorList &tensors, int tag) override { return Fallback(tensors)->recvAnysource(tensors, tag); }

private:
    static std::mutex &Mu()
    {
        static std::mutex m;
        return m;
    }
    static std::set<ProcessGroupZBAL *> &Live()
    {
        static std::set<ProcessGroupZBAL *> s;
        return s;
    }
    static std::map<std::tuple<int64_t, int64_t, int64_t>, int> &Counters()
    {
        static std::map<std::tuple<int64_t, int64_t, int64_t>, int> c;
        return c;
    }

    static bool OddBytes(const at::Tensor &t) { return ((uint64_t)t.numel() * t.element_size()) % 2 != 0; }
    static bool CudaReady() { return at::hasCUDA(); }

    bool UseZbal(const char *op, const TensorList &ts) const
    {
        if (forced_.count(op) || !strided_) return false;
        for (auto &t : ts)
            if (!t.is_cuda() || !t.is_contiguous()) return false;
        return true;
    }

    void DropFactory()
    {
        if (factory_ == nullptr) return;
        if (Py_IsInitialized()) {
            py::gil_scoped_acquire gil;
            delete factory_;
        }  // else: the interpreter is gone; the handle is left alone
        factory_ = nullptr;
    }

    c10::intrusive_ptr<c10d::Backend> Fallback(bool cuda)
    {
        auto &slot = cuda ? nccl_ : gloo_;
        if (!slot) {
            TORCH_CHECK(factory_ != nullptr, "zbal: this operation needs the ", cuda ? "NCCL" : "gloo", " fallback and no factory was set");
            py::gil_scoped_acquire gil;
            slot = (*factory_)(cuda).cast<c10::intrusive_ptr<c10d::Backend>>();
        }
        return slot;
    }
    c10::intrusive_ptr<c10d::Backend> Fallback(const TensorList &ts) { return Fallback(ts.empty() || ts[0].is_cuda()); }

    // Lazy bootstrap from the environment on the first collective, as the reference does.
    void EnsureInit()
    {
        if (zbal_is_bootstrapped()) return;
        zbal_bootstrap_options_t o;
        zbal_bootstrap_options_init(&o);
        std::string ipPort = EnvOr("ZBAL_IP_PORT", "");
        if (ipPort.empty())
            ipPort = EnvOr("MASTER_ADDR", "127.0.0.1") + ":" + std::to_string(std::stoi(EnvOr("MASTER_PORT", "29500")) + 7);
        if (ipPort.find("://") == std::string::npos) ipPort = "tcp://" + ipPort;
        TORCH_CHECK(ipPort.size() < sizeof(o.ipPort), "zbal: store address too long");
        std::snprintf(o.ipPort, sizeof(o.ipPort), "%s", ipPort.c_str());
        o.worldSize = (uint32_t)std::stoul(EnvOr("WORLD_SIZE", std::to_string(getSize()).c_str()));
        o.rankId = (uint32_t)std::stoul(EnvOr("RANK", std::to_string(getRank()).c_str()));
        o.deviceId = CudaReady() ? (int32_t)c10::cuda::current_device() : 0;
        o.startConfigServer = true;
        o.deviceMemorySize = std::stoull(EnvOr("ZBAL_DEVICE_MEM_SIZE", "4294967296"));
        if (CudaReady()) c10::cuda::device_synchronize();  // a context must exist before the VMM calls
        zbal_bootstrap_output_t out;
        Check(zbal_bootstrap(&o, &out), "zbal_bootstrap");
    }

    zbal_comm_t Communicator()
    {
        if (comm_ != nullptr) return comm_;
        TORCH_CHECK(strided_, "zbal: no communicator for a group of unevenly spaced ranks");
        EnsureInit();
        zbal_bootstrap_output_t out;
        Check(zbal_bootstrap_get_output(&out), "zbal_bootstrap_get_output");
        const int64_t first = ranks_.front(), last = ranks_.back(), step = getSize() > 1 ? ranks_[1] - first : 1;
        std::lock_guard<std::mutex> g(Mu());
        zbal_comm_t world = zbal_comm_get_global();
        if ((uint32_t)getSize() == out.worldSize && first == 0 && step == 1) {
            bool taken = false;
            for (auto *pg : Live()) taken = taken || (pg != this && pg->comm_ == world);
            if (!taken) return comm_ = world;
        }
        int n = Counters()[{first, last, step}]++;
        zbal_comm_options_t o{};
        std::snprintf(o.name, sizeof(o.name), "zbal_%ld:%ld:%ld_group_%d", (long)first, (long)last, (long)step, n);
        o.firstRank = (uint32_t)first;
        o.rankStep = (uint32_t)step;
        o.groupSize = (uint32_t)getSize();
        zbal_comm_t h = nullptr;
        Check(zbal_comm_create(&o, &h), o.name);
        return comm_ = h;
    }

    // (communicator of the pair, the peer's rank in it); created on first use, lower world rank is member 0.
    std::pair<zbal_comm_t, uint32_t> PairComm(int peerGroupRank)
    {
        TORCH_CHECK(peerGroupRank >= 0 && peerGroupRank < getSize() && peerGroupRank != getRank(), "zbal: bad peer rank ", peerGroupRank);
        const int64_t me = ranks_[getRank()], peer = ranks_[peerGroupRank], lo = std::min(me, peer), hi = std::max(me, peer);
        auto it = pairs_.find({lo, hi});
        if (it == pairs_.end()) {
            EnsureInit();
            std::string name = std::to_string(lo) + ":" + std::to_string(hi);
            zbal_comm_t h = zbal_comm_get_by_name(name.c_str());
            if (h == nullptr) {
                zbal_comm_options_t o{};
                std::snprintf(o.name, sizeof(o.name), "%s", name.c_str());
                o.firstRank = (uint32_t)lo;
                o.rankStep = (uint32_t)(hi - lo);
                o.groupSize = 2;
                Check(zbal_comm_create(&o, &h), name.c_str());
            }
            it = pairs_.emplace(std::make_pair(lo, hi), h).first;
        }
        return {it->second, me == lo ? 1u : 0u};
    }

    uint64_t StageBytes()
    {
        zbal_comm_property_t p{};
        Check(zbal_comm_get_property(Communicator(), &p), "zbal_comm_get_property");
        return p.stageBytes;
    }

    template <typename Fn>
    c10::intrusive_ptr<Work> Run(c10d::OpType op, const TensorList &touched, TensorList result, Fn &&fn)
    {
        seq_++;
        const c10::DeviceIndex dev = touched.empty() ? c10::cuda::current_device() : touched[0].device().index();
        c10::cuda::CUDAGuard devGuard(dev);
        c10::cuda::CUDAStream cur = c10::cuda::getCurrentCUDAStream(dev);
        auto done = std::make_shared<at::cuda::CUDAEvent>();
        if (!ownStream_) {
            fn(reinterpret_cast<zbal_stream_t>(cur.stream()));
            done->record(cur);
            return c10::make_intrusive<WorkZBAL>(getRank(), op, std::move(result), done, dev, TensorList{});
        }
        if (!stream_ || stream_->device_index() != dev) stream_ = c10::cuda::getStreamFromPool(false, dev);
        at::cuda::CUDAEvent ready;
        ready.record(cur);
        ready.block(*stream_);
        for (auto &t : touched) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), *stream_);
        {
            c10::cuda::CUDAStreamGuard sg(*stream_);  // tensor copies inside fn run on the side stream too
            fn(reinterpret_cast<zbal_stream_t>(stream_->stream()));
        }
        done->record(*stream_);
        return c10::make_intrusive<WorkZBAL>(getRank(), op, std::move(result), done, dev, touched);
    }

    c10::intrusive_ptr<c10d::Store> store_;
    std::vector<int64_t> ranks_;
    std::chrono::milliseconds timeout_;
    bool strided_ = true;
    bool ownStream_ = true;
    std::set<std::string> forced_;
    zbal_comm_t comm_ = nullptr;
    std::map<std::pair<int64_t, int64_t>, zbal_comm_t> pairs_;
    c10::intrusive_ptr<c10d::Backend> nccl_, gloo_;
    py::function *factory_ = nullptr;
    std::optional<c10::cuda::CUDAStream> stream_;
    uint64_t seq_ = 0;
};

void BindAllocator(py::module_ &m);  // zbal_torch_allocator.cpp

}  // namespace zbal_c10d

PYBIND11_MODULE(_zbal_c10d, m)
{
    using zbal_c10d::ProcessGroupZBAL;
    m.doc() = "zbal c10d backend (native)";
    py::class_<ProcessGroupZBAL, c10::intrusive_ptr<ProcessGroupZBAL>, c10d::Backend>(m, "ProcessGroupZBAL")
        .def(py::init([](const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, std::vector<int64_t> ranks,
                         std::chrono::milliseconds timeout) {
                 return c10::make_intrusive<ProcessGroupZBAL>(store, rank, size, std::move(ranks), timeout);
             }),
             py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("global_ranks") = std::vector<int64_t>{},
             py::arg("timeout") = std::chrono::milliseconds(30 * 60 * 1000), py::call_guard<py::gil_scoped_release>())
        .def("set_fallback_factory", &ProcessGroupZBAL::SetFallbackFactory)
        .def("device_status", &ProcessGroupZBAL::DeviceStatus, py::call_guard<py::gil_scoped_release>())
        .def("comm_name", &ProcessGroupZBAL::CommName, py::call_guard<py::gil_scoped_release>())
        .def("comm_handle", &ProcessGroupZBAL::CommHandle, py::call_guard<py::gil_scoped_release>())
        .def_property_readonly("strided", &ProcessGroupZBAL::Strided);
    m.def("forget_all", &ProcessGroupZBAL::ForgetAll);
    zbal_c10d::BindAllocator(m);
}
