// Operator classes with the method signatures of the reference's CL* operators
//   Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
//                     std::shared_ptr<Parameters> parameters);   // inputs = {ifm, weight, bias}, outputs = {ofm}
//   Status execute();   Status release();
// (CLConvolution.hpp:62-66, CLDepthwiseConvolution.hpp:33-38, CLDeconvolution.hpp:35-40, CLFullyConnected.hpp:30-35,
//  CLAdd.hpp, CLAveragepool.hpp), so OperationConstructor::create_ud_operator<OP> (gpu_op_constructor.cc:63-383) and
// EnnUDOperator<T>::execute (userdriver_operator.h:32-44) drive them exactly as they drive the OpenCL ones.
#pragma once
#include "b200_common.hpp"

namespace enn {
namespace ud {
namespace b200 {

// Shared implementation: translates tensors + parameters into a C-ABI descriptor, prepares once, executes on
// the device pointers the tensors hold at execute() time (buffers are assigned after all initialize() calls).
class B200OperatorBase {
public:
    B200OperatorBase(std::shared_ptr<B200Runtime> runtime, const PrecisionType &precision) : runtime_(std::move(runtime)), precision_(precision) {}
    virtual ~B200OperatorBase() { release(); }
    Status execute();
    Status release();
    // Device time of execute() (the per-operator bracket of userdriver_operator.h:35-42): off by default.
    Status setProfiling(bool on);
    Status lastExecuteMicroseconds(float *us);      // waits for the last execute() to finish
protected:
    Status run();
    Status prepare_conv_like(int kind, const enn_b200_conv_desc &desc, const std::shared_ptr<ITensor> &weight,
                             const std::shared_ptr<ITensor> &bias, const std::vector<float> &scales);
    Status ensure_nhwc_staging(bool nchw);
    std::shared_ptr<B200Runtime> runtime_;
    PrecisionType precision_;
    std::vector<std::shared_ptr<ITensor>> inputs_, outputs_;
    enn_b200_op *op_ = nullptr;
    bool nchw_ = false;
    Dim4 in_dim_{}, out_dim_{};          // logical NCHW-named dims (n, c, h, w)
    void *in_nhwc_ = nullptr, *out_nhwc_ = nullptr;
    bool two_inputs_ = false;
    bool runtime_weights_ = false, runtime_bias_ = false;   // filter / bias are not constant tensors
    enn_b200_timer *timer_ = nullptr;
};

class B200Convolution : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                      std::shared_ptr<Parameters> parameters);
};

class B200DepthwiseConvolution : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                      std::shared_ptr<Parameters> parameters);
};

class B200Deconvolution : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                      std::shared_ptr<Parameters> parameters);
};

class B200FullyConnected : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(const std::vector<std::shared_ptr<ITensor>> &input_tensors, const std::vector<std::shared_ptr<ITensor>> &output_tensors,
                      const std::shared_ptr<Parameters> parameters);
};

class B200Add : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                      std::shared_ptr<Parameters> parameters);
};

class B200Averagepool : public B200OperatorBase {
public:
    using B200OperatorBase::B200OperatorBase;
    Status initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                      std::shared_ptr<Parameters> parameters);
};

// The factory role of CLComputeLibrary::create* (CLComputeLibrary.hpp:23-107).
class B200ComputeLibrary {
public:
    explicit B200ComputeLibrary(int device = 0) : runtime_(std::make_shared<B200Runtime>(device)) {}
    std::shared_ptr<B200Runtime> runtime() const { return runtime_; }
    std::shared_ptr<ITensor> create_tensor(DataType type, const Dim4 &dim, DataOrder order, float scale, int32_t zero_point) {
        return std::make_shared<B200Tensor>(runtime_, type, dim, order, scale, zero_point, false);
    }
    std::shared_ptr<ITensor> create_and_copy_tensor(DataType type, const void *data, const Dim4 &dim, DataOrder order, float scale,
                                                    int32_t zero_point) {
        auto t = std::make_shared<B200Tensor>(runtime_, type, dim, order, scale, zero_point, true);
        t->writeData(const_cast<void *>(data));   // DataPtr is void * (Common.hpp:12); the bytes are only read
        return t;
    }
    std::shared_ptr<B200Convolution> createConvolution(const PrecisionType &p) { return std::make_shared<B200Convolution>(runtime_, p); }
    std::shared_ptr<B200DepthwiseConvolution> createDepthwiseConvolution(const PrecisionType &p) { return std::make_shared<B200DepthwiseConvolution>(runtime_, p); }
    std::shared_ptr<B200Deconvolution> createDeconvolution(const PrecisionType &p) { return std::make_shared<B200Deconvolution>(runtime_, p); }
    std::shared_ptr<B200FullyConnected> createFullyConnected(const PrecisionType &p) { return std::make_shared<B200FullyConnected>(runtime_, p); }
    std::shared_ptr<B200Add> createAdd(const PrecisionType &p) { return std::make_shared<B200Add>(runtime_, p); }
    std::shared_ptr<B200Averagepool> createAveragepool(const PrecisionType &p) { return std::make_shared<B200Averagepool>(runtime_, p); }
    Status synchronize() { return runtime_->synchronize(); }
private:
    std::shared_ptr<B200Runtime> runtime_;
};

}  // namespace b200
}  // namespace ud
}  // namespace enn
