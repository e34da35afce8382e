// MoELayerPlugin / MoELayerPluginCreator: the TensorRT-facing classes of the MoE layer.
//
// Same class names, plugin type/version strings, attribute names and virtual overrides as the reference
// (plugin/MoELayerPlugin.h:18-19,91-154); every body forwards to the C ABI of include/infmoe_c.h, so this
// file holds no arithmetic and no CUDA code.
#pragma once

#include <array>
#include <memory>
#include <string>

#include "infmoe_c.h"
#include "trt_compat.h"

namespace infmoe_plugin {
constexpr const char* kPluginName = "MoELayerPlugin";
constexpr const char* kPluginVersion = "1";
}  // namespace infmoe_plugin

class MoELayerPlugin : public nvinfer1::IPluginV2DynamicExt {
   public:
    // takes ownership of `layer`
    MoELayerPlugin(const char* layerName, infmoe_layer* layer);
    ~MoELayerPlugin() override;

    // IPluginV2
    const char* getPluginType() const noexcept override { return infmoe_plugin::kPluginName; }
    const char* getPluginVersion() const noexcept override { return infmoe_plugin::kPluginVersion; }
    int32_t getNbOutputs() const noexcept override { return 1; }
    int32_t initialize() noexcept override;
    void terminate() noexcept override;
    size_t getSerializationSize() const noexcept override;
    void serialize(void* buffer) const noexcept override;
    void destroy() noexcept override;
    void setPluginNamespace(const char* pluginNamespace) noexcept override;
    const char* getPluginNamespace() const noexcept override;
    // IPluginV2Ext
    nvinfer1::DataType getOutputDataType(int32_t index, const nvinfer1::DataType* inputTypes,
                                         int32_t nbInputs) const noexcept override;
    // IPluginV2DynamicExt
    nvinfer1::IPluginV2DynamicExt* clone() const noexcept override;
    nvinfer1::DimsExprs getOutputDimensions(int32_t outputIndex, const nvinfer1::DimsExprs* inputs, int32_t nbInputs,
                                            nvinfer1::IExprBuilder& exprBuilder) noexcept override;
    bool supportsFormatCombination(int32_t pos, const nvinfer1::PluginTensorDesc* inOut, int32_t nbInputs,
                                   int32_t nbOutputs) noexcept override;
    void configurePlugin(const nvinfer1::DynamicPluginTensorDesc* in, int32_t nbInputs,
                         const nvinfer1::DynamicPluginTensorDesc* out, int32_t nbOutputs) noexcept override;
    size_t getWorkspaceSize(const nvinfer1::PluginTensorDesc* inputs, int32_t nbInputs,
                            const nvinfer1::PluginTensorDesc* outputs, int32_t nbOutputs) const noexcept override;
    int32_t enqueue(const nvinfer1::PluginTensorDesc* inputDesc, const nvinfer1::PluginTensorDesc* outputDesc,
                    const void* const* inputs, void* const* outputs, void* workspace,
                    cudaStream_t stream) noexcept override;

    infmoe_layer* layer() const { return mLayer; }
    int sequenceLength() const { return mSequenceLength; }

    // One rank's share of an expert-parallel layer (INFMOE_EP_WORLD > 1): the layer object holding this rank's
    // experts and its wrapper.  Shared by the clones of a plugin: the communicator is one per process.
    struct Sharded {
        infmoe_layer* local = nullptr;
        infmoe_ep* ep = nullptr;
        ~Sharded();
    };

   private:
    std::string mLayerName, mNamespace;
    infmoe_layer* mLayer = nullptr;   // the whole layer's attributes; also the compute object when one GPU runs it
    std::shared_ptr<Sharded> mSharded;
    int mEmbeddingSize = 0;
    int mSequenceLength = -1;  // learnt in configurePlugin, like the reference (MoELayerPlugin.cc:170-180)
    int64_t mMaxTokens = 0;    // largest batch * seq_len configurePlugin announced
};

class MoELayerPluginCreator : public nvinfer1::IPluginCreator {
   public:
    MoELayerPluginCreator() = default;
    const char* getPluginName() const noexcept override { return infmoe_plugin::kPluginName; }
    const char* getPluginVersion() const noexcept override { return infmoe_plugin::kPluginVersion; }
    const nvinfer1::PluginFieldCollection* getFieldNames() noexcept override;
    nvinfer1::IPluginV2* createPlugin(const char* name, const nvinfer1::PluginFieldCollection* fc) noexcept override;
    nvinfer1::IPluginV2* deserializePlugin(const char* name, const void* serialData,
                                           size_t serialLength) noexcept override;
    void setPluginNamespace(const char* pluginNamespace) noexcept override;
    const char* getPluginNamespace() const noexcept override;

   private:
    std::string mNamespace;
};
