// Host-side mirror of the userdriver operator interface for the B200 library.
//
// Two build modes:
//  * inside the reference tree (-DENN_B200_WITH_REFERENCE_HEADERS, the reference's src/ and OpenCL stub directories on
//    the include path) the reference's own declarations are used:
//      userdriver/common/operator_interfaces/common/Common.hpp      (Status, Dim4, Dim2, Pad4, DataType, PrecisionType, ...)
//      userdriver/common/operator_interfaces/common/ActivationInfo.hpp
//      userdriver/common/operator_interfaces/interfaces/ITensor.hpp
//      userdriver/gpu/common/CLParameter.hpp                         (Parameters, Pool2DParameters)
//      userdriver/gpu/operators/CL{Convolution,DepthwiseConvolution,Deconvolution,FullyConnected,Add}.hpp (parameter structs)
//  * stand-alone, the declarations below stand in for them, with the same names, fields and meaning, so that
//    operator-construction code written against the OpenCL driver reads the same against this one.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/enn_b200.h"

#ifdef ENN_B200_WITH_REFERENCE_HEADERS
#include "userdriver/common/operator_interfaces/common/ActivationInfo.hpp"
#include "userdriver/common/operator_interfaces/common/Common.hpp"
#include "userdriver/common/operator_interfaces/interfaces/ITensor.hpp"
#include "userdriver/gpu/common/CLParameter.hpp"
#include "userdriver/gpu/operators/CLAdd.hpp"
#include "userdriver/gpu/operators/CLConvolution.hpp"
#include "userdriver/gpu/operators/CLDeconvolution.hpp"
#include "userdriver/gpu/operators/CLDepthwiseConvolution.hpp"
#include "userdriver/gpu/operators/CLFullyConnected.hpp"
#define ENN_B200_ITENSOR_OVERRIDE override
#else
#define ENN_B200_ITENSOR_OVERRIDE
#endif

namespace enn {
namespace ud {
namespace b200 {

#ifdef ENN_B200_WITH_REFERENCE_HEADERS
using ::ActivationInfo;
using ::DataOrder;
using ::DataOrderChangeType;
using ::DataPtr;
using ::DataType;
using ::Dim2;
using ::Dim4;
using ::enn::ud::ITensor;
using ::NDims;
using ::Pad4;
using ::PrecisionType;
using ::Status;
using ::StorageType;
using ::enn::ud::gpu::AddParameters;
using ::enn::ud::gpu::ConvolutionParameters;
using ::enn::ud::gpu::DeconvolutionParameters;
using ::enn::ud::gpu::DepthwiseConvolutionParameters;
using ::enn::ud::gpu::FullyConnectedParameters;
using ::enn::ud::gpu::Parameters;
using ::enn::ud::gpu::Pool2DParameters;
#else
typedef void *DataPtr;
typedef std::vector<uint32_t> NDims;
enum class Status { SUCCESS = 0, FAILURE = 1, CL_FAILURE = 2, INVALID_PARAMS = 3 };
enum class DataOrder { NCHW = 0, NHWC = 1, OTHER = 2 };
enum class DataOrderChangeType { NHWC2NCHW = 0, NCHW2NHWC = 1, NHWC2DHWC4 = 2, NCHW2DHWC4 = 3, DHWC42NHWC = 4, DHWC42NCHW = 5, OTHER = 6 };
enum class DataType { UNKNOWN = -1, FLOAT = 0, HALF = 1, INT32 = 2, INT8 = 3, UINT8 = 4, BOOL = 5, INT16 = 6, UINT16 = 7, FLOAT16 = 8 };
enum class PrecisionType { FP32 = 0, FP16 = 1, INT32 = 2, INT16 = 3, INT8 = 4, UINT8 = 5 };
enum class StorageType { BUFFER = 0, TEXTURE = 1 };
enum class ComputeType { TFLite = 0, Caffe };

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

// The accessors of ITensor (interfaces/ITensor.hpp:12-60) the quantized operators rely on; B200Tensor below implements
// the whole interface in either mode.
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
    virtual Status readData(DataPtr data, bool blocking = true, DataOrderChangeType type = DataOrderChangeType::OTHER, void *event = nullptr) = 0;
    virtual Status writeData(DataPtr data, bool blocking = true, DataOrderChangeType type = DataOrderChangeType::OTHER) = 0;
};
#endif

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

// Device tensor: dims + type + (scale, zero point) + a device allocation (the role of CLTensor,
// gpu/common/CLTensor.hpp); implements every member of ITensor.
class B200Tensor : public ITensor {
public:
    B200Tensor(std::shared_ptr<B200Runtime> rt, DataType type, const Dim4 &dim, DataOrder order = DataOrder::NCHW, float scale = 1.0f,
               int32_t zero_point = 0, bool is_const = false)
        : rt_(std::move(rt)), type_(type), dim_(dim), dims_{dim.n, dim.c, dim.h, dim.w}, order_(order), scale_(scale), zp_(zero_point),
          const_(is_const) {
        bytes_ = static_cast<size_t>(dim.n) * dim.c * dim.h * dim.w * elem_size();
        allocate();
    }
    ~B200Tensor() override { drop(); }
    size_t getNumOfBytes() ENN_B200_ITENSOR_OVERRIDE { return bytes_; }
    DataType getDataType() ENN_B200_ITENSOR_OVERRIDE { return type_; }
    PrecisionType getPrecisionType() ENN_B200_ITENSOR_OVERRIDE {
        switch (type_) {
            case DataType::UINT8: return PrecisionType::UINT8;
            case DataType::INT8: return PrecisionType::INT8;
            case DataType::INT32: return PrecisionType::INT32;
            case DataType::INT16: return PrecisionType::INT16;
            case DataType::HALF: case DataType::FLOAT16: return PrecisionType::FP16;
            default: return PrecisionType::FP32;
        }
    }
    const Dim4 &getDim() ENN_B200_ITENSOR_OVERRIDE { return dim_; }
    const NDims &getDims() ENN_B200_ITENSOR_OVERRIDE { return dims_; }
    uint32_t getDims(const int32_t &idx) ENN_B200_ITENSOR_OVERRIDE {
        const int32_t n = static_cast<int32_t>(dims_.size());
        const int32_t i = idx < 0 ? idx + n : idx;      // negative indices count from the end (CLTensor.hpp getDims(idx))
        return i >= 0 && i < n ? dims_[i] : 0;
    }
    uint32_t getNumOfDims() ENN_B200_ITENSOR_OVERRIDE { return static_cast<uint32_t>(dims_.size()); }
    uint32_t getTotalSizeFromDims() ENN_B200_ITENSOR_OVERRIDE {
        uint32_t t = 1;
        for (uint32_t d : dims_) t *= d;
        return t;
    }
    DataOrder getDataOrder() ENN_B200_ITENSOR_OVERRIDE { return order_; }
    float getScale() ENN_B200_ITENSOR_OVERRIDE { return scale_; }
    int32_t getZeroPoint() ENN_B200_ITENSOR_OVERRIDE { return zp_; }
    void setZeroPoint(int32_t zero_point) ENN_B200_ITENSOR_OVERRIDE { zp_ = zero_point; }
    void setScale(float scale) ENN_B200_ITENSOR_OVERRIDE { scale_ = scale; }
    void set_buffer_index(int32_t index) ENN_B200_ITENSOR_OVERRIDE { buffer_index_ = index; }
    int32_t get_buffer_index() ENN_B200_ITENSOR_OVERRIDE { return buffer_index_; }
    void set_buffer_type(uint32_t type) ENN_B200_ITENSOR_OVERRIDE { buffer_type_ = type; }
    uint32_t get_buffer_type() ENN_B200_ITENSOR_OVERRIDE { return buffer_type_; }
    // The executor hands pooled activation memory to a tensor after every initialize() has run
    // (gpu_op_constructor.cc:1839-1843); the tensor then stops owning an allocation of its own.
    void set_buffer_ptr(void *addr) ENN_B200_ITENSOR_OVERRIDE {
        drop();
        dev_ = addr;
        owned_ = false;
    }
    bool is_const() override { return const_; }

    Status writeData(DataPtr data, bool blocking = true, DataOrderChangeType type = DataOrderChangeType::OTHER) override {
        if (!data || !dev_) return Status::INVALID_PARAMS;
        host_copy_.resize(bytes_);
        if (!reordered(static_cast<const uint8_t *>(data), host_copy_.data(), type)) return Status::INVALID_PARAMS;
        Status s = to_status(enn_b200_upload(rt_->context(), dev_, host_copy_.data(), bytes_));
        if (s == Status::SUCCESS && blocking) s = rt_->synchronize();
        return s;
    }
    Status readData(DataPtr data, bool = true, DataOrderChangeType type = DataOrderChangeType::OTHER, void * = nullptr) override {
        if (!data || !dev_) return Status::INVALID_PARAMS;
        if (type == DataOrderChangeType::OTHER) return to_status(enn_b200_download(rt_->context(), data, dev_, bytes_));
        std::vector<uint8_t> tmp(bytes_);
        Status s = to_status(enn_b200_download(rt_->context(), tmp.data(), dev_, bytes_));
        if (s != Status::SUCCESS) return s;
        return reordered(tmp.data(), static_cast<uint8_t *>(data), type) ? Status::SUCCESS : Status::INVALID_PARAMS;
    }

    Status reconfigure(const PrecisionType &precision, const DataOrder &order, const Dim4 &dims, const float &scale,
                       const int32_t &offset) ENN_B200_ITENSOR_OVERRIDE {
        return reconfigure(precision, order, NDims{dims.n, dims.c, dims.h, dims.w}, scale, offset);
    }
    Status reconfigure(const PrecisionType &precision, const DataOrder &order, const NDims &ndim, const float &scale,
                       const int32_t &offset) ENN_B200_ITENSOR_OVERRIDE {
        if (precision == PrecisionType::UINT8) type_ = DataType::UINT8;
        else if (precision == PrecisionType::INT8) type_ = DataType::INT8;
        else if (precision == PrecisionType::INT32) type_ = DataType::INT32;
        else return Status::INVALID_PARAMS;            // this driver carries quantized tensors only
        order_ = order;
        scale_ = scale;
        zp_ = offset;
        return reconfigureDimsAndBuffer(ndim);
    }
    Status reconfigureDim(const Dim4 &dims) ENN_B200_ITENSOR_OVERRIDE { return reconfigureDims(NDims{dims.n, dims.c, dims.h, dims.w}); }
    // New extents inside the memory the tensor already has.
    Status reconfigureDims(const NDims &ndim) ENN_B200_ITENSOR_OVERRIDE {
        size_t need = elem_size();
        for (uint32_t d : ndim) need *= d;
        if (need > capacity_ && owned_) return Status::INVALID_PARAMS;
        set_dims(ndim, need);
        return Status::SUCCESS;
    }
    Status reconfigureDimAndBuffer(const Dim4 &dims) ENN_B200_ITENSOR_OVERRIDE {
        return reconfigureDimsAndBuffer(NDims{dims.n, dims.c, dims.h, dims.w});
    }
    Status reconfigureDimsAndBuffer(const NDims &ndim) ENN_B200_ITENSOR_OVERRIDE {
        size_t need = elem_size();
        for (uint32_t d : ndim) need *= d;
        set_dims(ndim, need);
        if (owned_ && need > capacity_) {
            drop();
            return allocate();
        }
        return Status::SUCCESS;
    }
    // NCHW <-> NHWC on the device, in place of the reference's convertToNHWC / convertToNCHW kernels.
    Status reorder(const DataOrder &order) ENN_B200_ITENSOR_OVERRIDE {
        if (order == order_) return Status::SUCCESS;
        if (elem_size() != 1 || order == DataOrder::OTHER || order_ == DataOrder::OTHER || !dev_) return Status::INVALID_PARAMS;
        void *tmp = nullptr;
        if (enn_b200_malloc(rt_->context(), bytes_, &tmp) != ENN_B200_SUCCESS) return Status::CL_FAILURE;
        // dim_ always carries NCHW-named extents in the tensor's current order: an NHWC tensor stores {n, h, w, c}.
        int32_t st;
        if (order == DataOrder::NHWC) {
            st = enn_b200_nchw_to_nhwc(rt_->context(), dev_, tmp, dim_.n, dim_.c, dim_.h, dim_.w);
            if (st == ENN_B200_SUCCESS) set_dims(NDims{dim_.n, dim_.h, dim_.w, dim_.c}, bytes_);
        } else {
            st = enn_b200_nhwc_to_nchw(rt_->context(), dev_, tmp, dim_.n, dim_.w, dim_.c, dim_.h);
            if (st == ENN_B200_SUCCESS) set_dims(NDims{dim_.n, dim_.w, dim_.c, dim_.h}, bytes_);
        }
        if (st == ENN_B200_SUCCESS) st = enn_b200_copy_device(rt_->context(), dev_, tmp, bytes_);
        if (st == ENN_B200_SUCCESS) st = enn_b200_stream_sync(rt_->context());     // tmp is freed below
        enn_b200_free(rt_->context(), tmp);
        if (st == ENN_B200_SUCCESS) order_ = order;
        return to_status(st);
    }
    void queryTensorInfo() ENN_B200_ITENSOR_OVERRIDE {
        std::printf("B200Tensor dims {%u, %u, %u, %u} order %d type %d scale %g zero point %d bytes %zu\n", dim_.n, dim_.c, dim_.h, dim_.w,
                    static_cast<int>(order_), static_cast<int>(type_), scale_, zp_, bytes_);
    }
    void dumpTensorData(std::string file_name) ENN_B200_ITENSOR_OVERRIDE {
        std::vector<uint8_t> tmp(bytes_);
        if (readData(tmp.data()) != Status::SUCCESS) return;
        if (FILE *f = std::fopen(file_name.c_str(), "wb")) {
            std::fwrite(tmp.data(), 1, tmp.size(), f);
            std::fclose(f);
        }
    }
    Status resetInterBuffer() ENN_B200_ITENSOR_OVERRIDE { return Status::SUCCESS; }

    // Device address (CLTensor::getDataPtr returns the cl_mem); operators cast to B200Tensor the way the OpenCL
    // operators cast to CLTensor.
    void *getDataPtr() const { return dev_; }
    // Constant tensors keep their host bytes: the operators re-pack weights on the host at initialize().
    const std::vector<uint8_t> &hostCopy() const { return host_copy_; }

private:
    size_t elem_size() const {
        switch (type_) {
            case DataType::INT32: case DataType::FLOAT: return 4;
            case DataType::HALF: case DataType::FLOAT16: case DataType::INT16: case DataType::UINT16: return 2;
            default: return 1;
        }
    }
    Status allocate() {
        owned_ = true;
        capacity_ = bytes_;
        return to_status(enn_b200_malloc(rt_->context(), bytes_ ? bytes_ : 1, &dev_));
    }
    void drop() {
        if (dev_ && owned_) enn_b200_free(rt_->context(), dev_);
        dev_ = nullptr;
        capacity_ = 0;
    }
    void set_dims(const NDims &ndim, size_t bytes) {
        dims_ = ndim;
        uint32_t d4[4] = {1, 1, 1, 1};
        for (size_t i = 0; i < ndim.size() && i < 4; ++i) d4[i] = ndim[i];
        dim_ = Dim4{d4[0], d4[1], d4[2], d4[3]};
        bytes_ = bytes;
    }
    // Host-side NCHW <-> NHWC of the tensor's bytes for readData / writeData; `type` names the change applied to the
    // caller's data on its way in (writeData) or out (readData).
    bool reordered(const uint8_t *src, uint8_t *dst, DataOrderChangeType type) const {
        if (type == DataOrderChangeType::OTHER) {
            std::memcpy(dst, src, bytes_);
            return true;
        }
        if (type != DataOrderChangeType::NHWC2NCHW && type != DataOrderChangeType::NCHW2NHWC) return false;
        const size_t e = elem_size();
        // dim_ names the extents as (n, c, h, w) of the logical tensor
        const size_t N = dim_.n, Cc = dim_.c, H = dim_.h, W = dim_.w;
        for (size_t n = 0; n < N; ++n)
            for (size_t c = 0; c < Cc; ++c)
                for (size_t h = 0; h < H; ++h)
                    for (size_t w = 0; w < W; ++w) {
                        const size_t nchw = ((n * Cc + c) * H + h) * W + w, nhwc = ((n * H + h) * W + w) * Cc + c;
                        const size_t s = type == DataOrderChangeType::NHWC2NCHW ? nhwc : nchw;
                        const size_t d = type == DataOrderChangeType::NHWC2NCHW ? nchw : nhwc;
                        std::memcpy(dst + d * e, src + s * e, e);
                    }
        return true;
    }
    std::shared_ptr<B200Runtime> rt_;
    DataType type_;
    Dim4 dim_;
    NDims dims_;
    DataOrder order_;
    float scale_;
    int32_t zp_;
    bool const_;
    size_t bytes_ = 0, capacity_ = 0;
    void *dev_ = nullptr;
    bool owned_ = true;
    int32_t buffer_index_ = -1;
    uint32_t buffer_type_ = 0;
    std::vector<uint8_t> host_copy_;
};

inline void *device_ptr(const std::shared_ptr<ITensor> &t) {
    auto bt = std::dynamic_pointer_cast<B200Tensor>(t);
    return bt ? bt->getDataPtr() : nullptr;
}

#ifndef ENN_B200_WITH_REFERENCE_HEADERS
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

// CLAdd.hpp:19-26
struct AddParameters : public Parameters {
    ActivationInfo activation_info = ActivationInfo();
    bool pot_scale_int16 = false;
    std::vector<float> coeff = {};
    bool androidNN = false;
    bool isNCHW = false;
    StorageType storage_type = StorageType::BUFFER;
};

// gpu/common/CLParameter.hpp:26-35
struct Pool2DParameters : public Parameters {
    Pad4 padding = {0, 0, 0, 0};
    Dim2 stride = {1, 1};
    Dim2 filter = {1, 1};
    ActivationInfo activation_info = ActivationInfo();
    bool androidNN = false;
    bool isNCHW = true;
    StorageType storage_type = StorageType::BUFFER;
    ComputeType compute_type = ComputeType::TFLite;
};
#endif   // !ENN_B200_WITH_REFERENCE_HEADERS

}  // namespace b200
}  // namespace ud
}  // namespace enn
