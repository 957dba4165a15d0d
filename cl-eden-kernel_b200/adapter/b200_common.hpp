// Host-side mirror of the userdriver operator interface for the B200 library.
//
// The types below carry the same names, fields and meaning as the reference's
//   userdriver/common/operator_interfaces/common/Common.hpp      (Status, Dim4, Dim2, Pad4, DataType, PrecisionType, DataOrder)
//   userdriver/common/operator_interfaces/common/ActivationInfo.hpp
//   userdriver/common/operator_interfaces/interfaces/ITensor.hpp (the accessors the quantized operators use)
//   userdriver/gpu/common/CLParameter.hpp                         (Parameters base)
// so that operator-construction code written against the OpenCL driver reads the same against this one.
// Inside the reference tree these declarations are replaced by the reference's own headers.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "../../include/enn_b200.h"

namespace enn {
namespace ud {
namespace b200 {

enum class Status { SUCCESS = 0, FAILURE = 1, CL_FAILURE = 2, INVALID_PARAMS = 3 };
enum class DataOrder { NCHW = 0, NHWC = 1, OTHER = 2 };
enum class DataType { UNKNOWN = -1, FLOAT = 0, HALF = 1, INT32 = 2, INT8 = 3, UINT8 = 4 };
enum class PrecisionType { FP32 = 0, FP16 = 1, INT32 = 2, INT16 = 3, INT8 = 4, UINT8 = 5 };
enum class StorageType { BUFFER = 0, TEXTURE = 1 };

struct Dim4 { uint32_t n, c, h, w; };
struct Dim2 { uint32_t h, w; };
struct Pad4 { uint32_t t, r, b, l; };

class ActivationInfo {
public:
    enum class ActivationType { NONE, RELU, RELU1, RELU6, TANH, SIGMOID };
    ActivationInfo() = default;
    ActivationInfo(ActivationType type, const bool &enabled) : type_(type), enabled_(enabled) {}
    ActivationType activation() const { return type_; }
    bool isEnabled() const { return enabled_; }
private:
    ActivationType type_ = ActivationType::NONE;
    bool enabled_ = false;
};

inline Status to_status(int32_t s) { return static_cast<Status>(s); }

// One device + one stream: the role CLRuntime plays for the OpenCL operators.
class B200Runtime {
public:
    explicit B200Runtime(int device = 0) { status_ = to_status(enn_b200_context_create(device, &ctx_)); }
    ~B200Runtime() { if (ctx_) enn_b200_context_destroy(ctx_); }
    B200Runtime(const B200Runtime &) = delete;
    B200Runtime &operator=(const B200Runtime &) = delete;
    Status status() const { return status_; }
    enn_b200_context *context() const { return ctx_; }
    Status synchronize() { return to_status(enn_b200_stream_sync(ctx_)); }
    std::string lastError() const {
        char buf[256];
        enn_b200_last_error(ctx_, buf, sizeof(buf));
        return buf;
    }
private:
    enn_b200_context *ctx_ = nullptr;
    Status status_ = Status::FAILURE;
};

// The accessors of ITensor (interfaces/ITensor.hpp:14-37) the quantized operators rely on.
class ITensor {
public:
    virtual ~ITensor() = default;
    virtual size_t getNumOfBytes() = 0;
    virtual DataType getDataType() = 0;
    virtual const Dim4 &getDim() = 0;
    virtual DataOrder getDataOrder() = 0;
    virtual float getScale() = 0;
    virtual int32_t getZeroPoint() = 0;
    virtual bool is_const() { return false; }
    virtual Status readData(void *data, bool blocking = true) = 0;
    virtual Status writeData(const void *data, bool blocking = true) = 0;
    virtual void *getDataPtr() = 0;   // device pointer (CLTensor::getDataPtr returns the cl_mem)
};

// Device tensor: dims + type + (scale, zero point) + a device allocation (CLTensor, gpu/common/CLTensor.hpp).
class B200Tensor : public ITensor {
public:
    B200Tensor(std::shared_ptr<B200Runtime> rt, DataType type, const Dim4 &dim, DataOrder order = DataOrder::NCHW, float scale = 1.0f,
               int32_t zero_point = 0, bool is_const = false)
        : rt_(std::move(rt)), type_(type), dim_(dim), order_(order), scale_(scale), zp_(zero_point), const_(is_const) {
        const size_t elem = (type == DataType::INT32 || type == DataType::FLOAT) ? 4 : (type == DataType::HALF ? 2 : 1);
        bytes_ = static_cast<size_t>(dim.n) * dim.c * dim.h * dim.w * elem;
        enn_b200_malloc(rt_->context(), bytes_, &dev_);
    }
    ~B200Tensor() override { if (dev_) enn_b200_free(rt_->context(), dev_); }
    size_t getNumOfBytes() override { return bytes_; }
    DataType getDataType() override { return type_; }
    const Dim4 &getDim() override { return dim_; }
    DataOrder getDataOrder() override { return order_; }
    float getScale() override { return scale_; }
    int32_t getZeroPoint() override { return zp_; }
    bool is_const() override { return const_; }
    Status writeData(const void *data, bool blocking = true) override {
        host_copy_.assign(static_cast<const uint8_t *>(data), static_cast<const uint8_t *>(data) + bytes_);
        Status s = to_status(enn_b200_upload(rt_->context(), dev_, host_copy_.data(), bytes_));
        if (s == Status::SUCCESS && blocking) s = rt_->synchronize();
        return s;
    }
    Status readData(void *data, bool = true) override { return to_status(enn_b200_download(rt_->context(), data, dev_, bytes_)); }
    void *getDataPtr() override { return dev_; }
    // Constant tensors keep their host bytes: the operators re-pack weights on the host at initialize().
    const std::vector<uint8_t> &hostCopy() const { return host_copy_; }
private:
    std::shared_ptr<B200Runtime> rt_;
    DataType type_;
    Dim4 dim_;
    DataOrder order_;
    float scale_;
    int32_t zp_;
    bool const_;
    size_t bytes_ = 0;
    void *dev_ = nullptr;
    std::vector<uint8_t> host_copy_;
};

struct Parameters {
    virtual ~Parameters() = default;
};

// CLConvolution.hpp:31-44
struct ConvolutionParameters : public Parameters {
    Pad4 padding = {0, 0, 0, 0};
    Dim2 dilation = {1, 1};
    Dim2 stride = {1, 1};
    uint32_t group_size = 1;
    uint32_t axis = 0;
    bool per_channel_quant = false;
    bool androidNN = false;
    bool isNCHW = true;
    StorageType storage_type = StorageType::BUFFER;
    bool openAibWino = false;
    std::shared_ptr<ActivationInfo> activation_info = std::make_shared<ActivationInfo>();
    std::vector<float> scales;
};

// CLDepthwiseConvolution.hpp:18-29
struct DepthwiseConvolutionParameters : public Parameters {
    Pad4 padding = {0, 0, 0, 0};
    Dim2 dilation = {1, 1};
    Dim2 stride = {1, 1};
    uint32_t depth_multiplier = 1;
    bool per_channel_quant = false;
    bool androidNN = false;
    bool isNCHW = true;
    StorageType storage_type = StorageType::BUFFER;
    std::shared_ptr<ActivationInfo> activation_info = std::make_shared<ActivationInfo>();
    std::vector<float> scales;
};

// CLDeconvolution.hpp:20-31
struct DeconvolutionParameters : public Parameters {
    Pad4 padding = {0, 0, 0, 0};
    Dim2 stride = {1, 1};
    uint32_t group_size = 1;
    bool weights_as_input = false;
    bool per_channel_quant = false;
    bool androidNN = false;
    bool isNCHW = true;
    bool openAibWino = false;
    std::shared_ptr<ActivationInfo> activation_info = std::make_shared<ActivationInfo>();
    std::vector<float> scales;
};

// CLFullyConnected.hpp:21-25
struct FullyConnectedParameters : public Parameters {
    bool androidNN = false;
    StorageType storage_type = StorageType::BUFFER;
    std::shared_ptr<ActivationInfo> activation_info = std::make_shared<ActivationInfo>();
};

struct AddParameters : public Parameters {
    ActivationInfo activation_info;
};

struct Pool2DParameters : public Parameters {
    Pad4 padding = {0, 0, 0, 0};
    Dim2 stride = {1, 1};
    Dim2 filter = {1, 1};
    ActivationInfo activation_info;
};

}  // namespace b200
}  // namespace ud
}  // namespace enn
