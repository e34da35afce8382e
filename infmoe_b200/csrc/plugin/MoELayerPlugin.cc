// MoELayerPlugin: every TensorRT virtual forwards to the C ABI (reference bodies: plugin/MoELayerPlugin.cc).
#include "MoELayerPlugin.h"

#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>

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

int env_int(const char* name, int fallback) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : fallback;
}

// The communicator id of an expert-parallel run travels through a file every rank can see (INFMOE_EP_ID_FILE):
// rank 0 creates it (written under a temporary name and renamed, so a reader never sees half of it), the others
// wait for it to appear.
bool exchange_unique_id(int rank, const std::string& path, unsigned char* id) {
    if (rank == 0) {
        if (infmoe_ep_unique_id(id) != INFMOE_OK) return false;
        const std::string tmp = path + ".tmp";
        FILE* f = fopen(tmp.c_str(), "wb");
        if (!f) return false;
        const bool ok = fwrite(id, 1, INFMOE_EP_ID_BYTES, f) == INFMOE_EP_ID_BYTES;
        fclose(f);
        return ok && rename(tmp.c_str(), path.c_str()) == 0;
    }
    const int limit_s = env_int("INFMOE_EP_ID_TIMEOUT_S", 120);
    for (int waited_ms = 0; waited_ms < limit_s * 1000; waited_ms += 50) {
        FILE* f = fopen(path.c_str(), "rb");
        if (f) {
            const bool ok = fread(id, 1, INFMOE_EP_ID_BYTES, f) == INFMOE_EP_ID_BYTES;
            fclose(f);
            if (ok) return true;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    return false;
}

}  // namespace

MoELayerPlugin::Sharded::~Sharded() {
    if (ep) infmoe_ep_destroy(ep);
    if (local) infmoe_layer_destroy(local);
}

MoELayerPlugin::MoELayerPlugin(const char* layerName, infmoe_layer* layer)
    : mLayerName(layerName ? layerName : ""), mLayer(layer) {
    infmoe_layer_config cfg{};
    if (mLayer && infmoe_layer_get_config(mLayer, &cfg) == INFMOE_OK) mEmbeddingSize = cfg.embedding_size;
}

MoELayerPlugin::~MoELayerPlugin() { terminate(); }

// One GPU: the reference's initialize (weights to pinned host memory).  Several GPUs (the reference has no such
// mode): INFMOE_EP_WORLD ranks, this process being INFMOE_EP_RANK, each with its own engine; this rank loads its
// expert_count / world experts from the weight file and joins the others (collective: every rank's plugin must
// reach this call).  Needs configurePlugin to have run (the receive buffers are sized by the largest batch).
int32_t MoELayerPlugin::initialize() noexcept {
    const int world = env_int("INFMOE_EP_WORLD", 1);
    if (world > 1) {
        if (mSharded) return 0;
        const int rank = env_int("INFMOE_EP_RANK", -1);
        const char* id_file = getenv("INFMOE_EP_ID_FILE");
        if (rank < 0 || rank >= world || !id_file || !*id_file || mMaxTokens <= 0) {
            fprintf(stderr, "ERROR: initialize: expert parallelism needs INFMOE_EP_RANK in [0, %d), INFMOE_EP_ID_FILE and a "
                            "configured plugin\n", world);
            return 1;
        }
        unsigned char id[INFMOE_EP_ID_BYTES];
        if (!exchange_unique_id(rank, id_file, id)) {
            fprintf(stderr, "ERROR: initialize: no communicator id through %s\n", id_file);
            return 1;
        }
        infmoe_layer_config whole{};
        auto sharded = std::make_shared<Sharded>();
        if (infmoe_layer_get_config(mLayer, &whole) != INFMOE_OK ||
            infmoe_ep_create_sharded(&whole, rank, world, id, mMaxTokens, &sharded->local, &sharded->ep) != INFMOE_OK) {
            report("initialize");
            return 1;
        }
        mSharded = sharded;
        return 0;
    }
    if (infmoe_layer_initialize(mLayer) != INFMOE_OK) {
        report("initialize");
        return 1;
    }
    return 0;
}

void MoELayerPlugin::terminate() noexcept {
    mSharded.reset();
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
    p->mMaxTokens = mMaxTokens;
    p->mSharded = mSharded;
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
    const int64_t batch = in[0].max.nbDims == 3 && in[0].max.d[0] > 0 ? in[0].max.d[0] : in[0].desc.dims.d[0];
    if (batch * mSequenceLength > mMaxTokens) mMaxTokens = batch * mSequenceLength;
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
    if (mSharded) {   // expert parallel: the wrapper owns its buffers, TensorRT's workspace is not used
        if (infmoe_ep_forward(mSharded->ep, static_cast<const float*>(inputs[0]), static_cast<float*>(outputs[0]), tokens,
                              stream) != INFMOE_OK) {
            report("enqueue");
            return 1;
        }
        return 0;
    }
    size_t bytes = 0;
    if (infmoe_layer_workspace_bytes(mLayer, tokens, &bytes) != INFMOE_OK ||
        infmoe_layer_enqueue(mLayer, static_cast<const float*>(inputs[0]), static_cast<float*>(outputs[0]), workspace,
                             bytes, tokens, stream) != INFMOE_OK) {
        report("enqueue");
        return 1;
    }
    return 0;
}
