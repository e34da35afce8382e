// The slice of TensorRT's plugin API that MoELayerPlugin / MoELayerPluginCreator use.
//
// When TensorRT's headers are installed the real <NvInferPlugin.h> is used and this file adds nothing.
// Without them (this project builds on machines that have CUDA but no TensorRT) the declarations below
// stand in, with the same names, members and virtual-function order as the public API for the classes
// the plugin derives from (IPluginV2 -> IPluginV2Ext -> IPluginV2DynamicExt, IPluginCreator), so that the
// plugin sources compile unchanged either way.  The stand-in also keeps a minimal creator registry so
// that REGISTER_TENSORRT_PLUGIN still registers the creator when the library is loaded.
#pragma once

#if defined(__has_include)
#if __has_include(<NvInferPlugin.h>)
#include <NvInferPlugin.h>
#define INFMOE_HAVE_TENSORRT 1
#endif
#endif

#ifndef INFMOE_HAVE_TENSORRT
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

struct cudnnContext;
struct cublasContext;

namespace nvinfer1 {

enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4 };
enum class TensorFormat : int32_t { kLINEAR = 0, kCHW2 = 1, kHWC8 = 2, kCHW4 = 3 };
using PluginFormat = TensorFormat;
enum class PluginFieldType : int32_t {
    kFLOAT16 = 0, kFLOAT32 = 1, kFLOAT64 = 2, kINT8 = 3, kINT16 = 4, kINT32 = 5, kCHAR = 6, kDIMS = 7, kUNKNOWN = 8
};

struct Dims {
    static constexpr int32_t MAX_DIMS = 8;
    int32_t nbDims;
    int32_t d[MAX_DIMS];
};

class IDimensionExpr;
struct DimsExprs {
    int32_t nbDims;
    const IDimensionExpr* d[Dims::MAX_DIMS];
};
class IExprBuilder;
class IGpuAllocator;

struct PluginTensorDesc {
    Dims dims;
    DataType type;
    TensorFormat format;
    float scale;
};
struct DynamicPluginTensorDesc {
    PluginTensorDesc desc;
    Dims min;
    Dims max;
};

struct PluginField {
    const char* name;
    const void* data;
    PluginFieldType type;
    int32_t length;
    PluginField(const char* n = nullptr, const void* d = nullptr, PluginFieldType t = PluginFieldType::kUNKNOWN,
                int32_t l = 0)
        : name(n), data(d), type(t), length(l) {}
};
struct PluginFieldCollection {
    int32_t nbFields;
    const PluginField* fields;
};

class IPluginV2 {
   public:
    virtual int32_t getTensorRTVersion() const noexcept { return 8000; }
    virtual const char* getPluginType() const noexcept = 0;
    virtual const char* getPluginVersion() const noexcept = 0;
    virtual int32_t getNbOutputs() const noexcept = 0;
    virtual int32_t initialize() noexcept = 0;
    virtual void terminate() noexcept = 0;
    virtual size_t getSerializationSize() const noexcept = 0;
    virtual void serialize(void* buffer) const noexcept = 0;
    virtual void destroy() noexcept = 0;
    virtual void setPluginNamespace(const char* pluginNamespace) noexcept = 0;
    virtual const char* getPluginNamespace() const noexcept = 0;
    virtual ~IPluginV2() = default;
};

class IPluginV2Ext : public IPluginV2 {
   public:
    virtual DataType getOutputDataType(int32_t index, const DataType* inputTypes, int32_t nbInputs) const noexcept = 0;
    virtual void attachToContext(cudnnContext*, cublasContext*, IGpuAllocator*) noexcept {}
    virtual void detachFromContext() noexcept {}
};

class IPluginV2DynamicExt : public IPluginV2Ext {
   public:
    virtual IPluginV2DynamicExt* clone() const noexcept = 0;
    virtual DimsExprs getOutputDimensions(int32_t outputIndex, const DimsExprs* inputs, int32_t nbInputs,
                                          IExprBuilder& exprBuilder) noexcept = 0;
    virtual bool supportsFormatCombination(int32_t pos, const PluginTensorDesc* inOut, int32_t nbInputs,
                                           int32_t nbOutputs) noexcept = 0;
    virtual void configurePlugin(const DynamicPluginTensorDesc* in, int32_t nbInputs,
                                 const DynamicPluginTensorDesc* out, int32_t nbOutputs) noexcept = 0;
    virtual size_t getWorkspaceSize(const PluginTensorDesc* inputs, int32_t nbInputs, const PluginTensorDesc* outputs,
                                    int32_t nbOutputs) const noexcept = 0;
    virtual int32_t enqueue(const PluginTensorDesc* inputDesc, const PluginTensorDesc* outputDesc,
                            const void* const* inputs, void* const* outputs, void* workspace,
                            cudaStream_t stream) noexcept = 0;
};

class IPluginCreator {
   public:
    virtual int32_t getTensorRTVersion() const noexcept { return 8000; }
    virtual const char* getPluginName() const noexcept = 0;
    virtual const char* getPluginVersion() const noexcept = 0;
    virtual const PluginFieldCollection* getFieldNames() noexcept = 0;
    virtual IPluginV2* createPlugin(const char* name, const PluginFieldCollection* fc) noexcept = 0;
    virtual IPluginV2* deserializePlugin(const char* name, const void* serialData, size_t serialLength) noexcept = 0;
    virtual void setPluginNamespace(const char* pluginNamespace) noexcept = 0;
    virtual const char* getPluginNamespace() const noexcept = 0;
    virtual ~IPluginCreator() = default;
};

// Stand-in registry: creators registered by REGISTER_TENSORRT_PLUGIN at load time.
void compatRegisterCreator(IPluginCreator* creator) noexcept;
IPluginCreator* compatGetCreator(const char* name, const char* version) noexcept;

template <typename T>
struct CompatRegistrar {
    T instance;
    CompatRegistrar() { compatRegisterCreator(&instance); }
};

}  // namespace nvinfer1

#define REGISTER_TENSORRT_PLUGIN(name) static nvinfer1::CompatRegistrar<name> pluginRegistrar##name {}
#endif  // !INFMOE_HAVE_TENSORRT
