// MoELayerPlugin: every TensorRT virtual forwards to the C ABI (reference bodies: plugin/MoELayerPlugin.cc).
#include "MoELayerPlugin.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

using namespace nvinfer1;

namespace {

// The reference prints and then asserts / exits on every failure (plugin/utility.h:15-21, README.md:86-94).
// Here the message is printed and the call fails; INFMOE_ABORT_ON_ERROR=1 restores the abort.
void report(const char* where) {
    fprintf(stderr, "ERROR: %s: %s\n", where, infmoe_last_error());
    const char* a = getenv("INFMOE_ABORT_ON_ERROR");
    if (a && *a == '1') abort();
}

int64_t token_count(const Dims& d, int seqLen) { return (int64_t)d.d[0] * (int64_t)seqLen; }

}  // namespace

MoELayerPlugin::MoELayerPlugin(const char* layerName, infmoe_layer* layer)
    : mLayerName(layerName ? layerName : ""), mLayer(layer) {
    infmoe_layer_config cfg{};
    if (mLayer && infmoe_layer_get_config(mLayer, &cfg) == INFMOE_OK) mEmbeddingSize = cfg.embedding_size;
}

MoELayerPlugin::~MoELayerPlugin() { terminate(); }

int32_t MoELayerPlugin::initialize() noexcept {
    if (infmoe_layer_initialize(mLayer) != INFMOE_OK) {
        report("initialize");
        return 1;
    }
    return 0;
}

void MoELayerPlugin::terminate() noexcept {
    if (mLayer) {
        infmoe_layer_destroy(mLayer);
        mLayer = nullptr;
    }
}

size_t MoELayerPlugin::getSerializationSize() const noexcept {
    size_t n = 0;
    if (infmoe_layer_serialization_size(mLayer, &n) != INFMOE_OK) report("getSerializationSize");
    return n;
}

void MoELayerPlugin::serialize(void* buffer) const noexcept {
    if (infmoe_layer_serialize(mLayer, buffer, getSerializationSize()) != INFMOE_OK) report("serialize");
}

// TensorRT calls destroy() on objects it also deletes through other paths; like the reference
// (plugin/MoELayerPlugin.cc:460-463) this is deliberately not a delete.
void MoELayerPlugin::destroy() noexcept {}

void MoELayerPlugin::setPluginNamespace(const char* pluginNamespace) noexcept {
    mNamespace = pluginNamespace ? pluginNamespace : "";
}
const char* MoELayerPlugin::getPluginNamespace() const noexcept { return mNamespace.c_str(); }

DataType MoELayerPlugin::getOutputDataType(int32_t, const DataType* inputTypes, int32_t) const noexcept {
    return inputTypes[0];
}

IPluginV2DynamicExt* MoELayerPlugin::clone() const noexcept {
    infmoe_layer* copy = nullptr;
    if (infmoe_layer_clone(mLayer, &copy) != INFMOE_OK) {
        report("clone");
        return nullptr;
    }
    auto* p = new MoELayerPlugin(mLayerName.c_str(), copy);
    p->mNamespace = mNamespace;
    p->mSequenceLength = mSequenceLength;
    return p;
}

// The output has the shape of the input (plugin/sublayers/T5FFLayer.cc:37-41).
DimsExprs MoELayerPlugin::getOutputDimensions(int32_t, const DimsExprs* inputs, int32_t, IExprBuilder&) noexcept {
    return inputs[0];
}

// FP32, linear layout only (plugin/MoELayerPlugin.cc:157-162).
bool MoELayerPlugin::supportsFormatCombination(int32_t pos, const PluginTensorDesc* inOut, int32_t nbInputs,
                                               int32_t nbOutputs) noexcept {
    if (nbInputs != 1 || nbOutputs != 1 || pos < 0 || pos > 1) return false;
    return inOut[pos].format == TensorFormat::kLINEAR && inOut[pos].type == DataType::kFLOAT;
}

// 3-D input [B, S, D] with D == embedding_size; S is remembered (plugin/MoELayerPlugin.cc:170-180).
void MoELayerPlugin::configurePlugin(const DynamicPluginTensorDesc* in, int32_t nbInputs,
                                     const DynamicPluginTensorDesc* out, int32_t nbOutputs) noexcept {
    (void)out;
    if (nbInputs != 1 || nbOutputs != 1 || in[0].desc.dims.nbDims != 3 || in[0].desc.dims.d[2] != mEmbeddingSize) {
        fprintf(stderr, "ERROR: configurePlugin: expected one 3-D input [batch, seq_len, %d]\n", mEmbeddingSize);
        const char* a = getenv("INFMOE_ABORT_ON_ERROR");
        if (a && *a == '1') abort();
        mSequenceLength = -1;
        return;
    }
    mSequenceLength = in[0].desc.dims.d[1];
}

size_t MoELayerPlugin::getWorkspaceSize(const PluginTensorDesc* inputs, int32_t nbInputs, const PluginTensorDesc*,
                                        int32_t nbOutputs) const noexcept {
    if (nbInputs != 1 || nbOutputs != 1 || inputs[0].dims.nbDims != 3 || mSequenceLength < 0) return 0;
    size_t bytes = 0;
    if (infmoe_layer_workspace_bytes(mLayer, token_count(inputs[0].dims, mSequenceLength), &bytes) != INFMOE_OK)
        report("getWorkspaceSize");
    return bytes;
}

int32_t MoELayerPlugin::enqueue(const PluginTensorDesc* inputDesc, const PluginTensorDesc*, const void* const* inputs,
                                void* const* outputs, void* workspace, cudaStream_t stream) noexcept {
    if (mSequenceLength < 0) {
        fprintf(stderr, "ERROR: enqueue: configurePlugin has not run\n");
        return 1;
    }
    const int64_t tokens = token_count(inputDesc[0].dims, mSequenceLength);
    size_t bytes = 0;
    if (infmoe_layer_workspace_bytes(mLayer, tokens, &bytes) != INFMOE_OK ||
        infmoe_layer_enqueue(mLayer, static_cast<const float*>(inputs[0]), static_cast<float*>(outputs[0]), workspace,
                             bytes, tokens, stream) != INFMOE_OK) {
        report("enqueue");
        return 1;
    }
    return 0;
}
