// MoELayerPluginCreator: the nine plugin attributes -> infmoe_layer_create.
// Reference: plugin/MoELayerPluginCreator.cc (attribute table :15-47, parsing :75-115, checks :118-140).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "MoELayerPlugin.h"

using namespace nvinfer1;

namespace {

const std::array<PluginField, 9>& attributeTable() {
    static const std::array<PluginField, 9> table = {
        PluginField{"expert_count", nullptr, PluginFieldType::kINT32, 1},
        PluginField{"embedding_size", nullptr, PluginFieldType::kINT32, 1},
        PluginField{"hidden_size", nullptr, PluginFieldType::kINT32, 1},
        PluginField{"max_concurrency", nullptr, PluginFieldType::kINT32, 1},
        PluginField{"expert_centroids", nullptr, PluginFieldType::kFLOAT32, 1},
        PluginField{"expert_weight_file", nullptr, PluginFieldType::kUNKNOWN, 1},
        PluginField{"expert_sublayer_type", nullptr, PluginFieldType::kUNKNOWN, 1},
        PluginField{"moe_variant", nullptr, PluginFieldType::kUNKNOWN, 1},
        PluginField{"layernorm_weight", nullptr, PluginFieldType::kFLOAT32, 1},
    };
    return table;
}

IPluginV2* fail(const char* fmt, const char* a = "", long b = 0) {
    fprintf(stderr, "ERROR: ");
    fprintf(stderr, fmt, a, b);
    fprintf(stderr, "\n");
    const char* ab = getenv("INFMOE_ABORT_ON_ERROR");
    if (ab && *ab == '1') abort();
    return nullptr;
}

}  // namespace

#ifndef INFMOE_HAVE_TENSORRT
namespace nvinfer1 {
namespace {
std::mutex& registryMutex() {
    static std::mutex m;
    return m;
}
std::vector<IPluginCreator*>& registry() {
    static std::vector<IPluginCreator*> r;
    return r;
}
}  // namespace
void compatRegisterCreator(IPluginCreator* creator) noexcept {
    std::lock_guard<std::mutex> lock(registryMutex());
    registry().push_back(creator);
}
IPluginCreator* compatGetCreator(const char* name, const char* version) noexcept {
    std::lock_guard<std::mutex> lock(registryMutex());
    for (IPluginCreator* c : registry())
        if (strcmp(c->getPluginName(), name) == 0 && strcmp(c->getPluginVersion(), version) == 0) return c;
    return nullptr;
}
}  // namespace nvinfer1
#endif

REGISTER_TENSORRT_PLUGIN(MoELayerPluginCreator);

const PluginFieldCollection* MoELayerPluginCreator::getFieldNames() noexcept {
    static const PluginFieldCollection fc{(int32_t)attributeTable().size(), attributeTable().data()};
    return &fc;
}

IPluginV2* MoELayerPluginCreator::createPlugin(const char* name, const PluginFieldCollection* fc) noexcept {
    if (!fc) return fail("createPlugin: no field collection");
    // defaults of the reference: T5_FF experts, cpm_2 variant, two weight slots (MoELayerPluginCreator.cc:62-66)
    int32_t expertCount = 0, embeddingSize = 0, hiddenSize = 0, maxConcurrency = 2;
    std::string weightFile, sublayerType = "T5_FF", variant = "cpm_2";
    const float* centroids = nullptr;
    const float* layernorm = nullptr;
    int32_t centroidLen = 0, layernormLen = 0;

    auto as_int = [](const PluginField& f, int32_t* out) {
        if (f.type != PluginFieldType::kINT32 || f.length != 1 || !f.data) return false;
        *out = *static_cast<const int32_t*>(f.data);
        return true;
    };
    for (int32_t i = 0; i < fc->nbFields; ++i) {
        const PluginField& f = fc->fields[i];
        const std::string key = f.name ? f.name : "";
        bool ok = true;
        if (key == "expert_count") ok = as_int(f, &expertCount);
        else if (key == "embedding_size") ok = as_int(f, &embeddingSize);
        else if (key == "hidden_size") ok = as_int(f, &hiddenSize);
        else if (key == "max_concurrency") ok = as_int(f, &maxConcurrency);
        else if (key == "expert_centroids") {
            ok = f.type == PluginFieldType::kFLOAT32 && f.data;
            centroids = static_cast<const float*>(f.data);
            centroidLen = f.length;
        } else if (key == "layernorm_weight") {
            ok = f.type == PluginFieldType::kFLOAT32 && f.data;
            layernorm = static_cast<const float*>(f.data);
            layernormLen = f.length;
        } else if (key == "expert_weight_file" || key == "expert_sublayer_type" || key == "moe_variant") {
            // character data of `length` bytes, not necessarily terminated
            ok = f.data != nullptr;
            if (ok) {
                const char* p = static_cast<const char*>(f.data);
                std::string v(p, strnlen(p, (size_t)(f.length > 0 ? f.length : 0)));
                if (key == "expert_weight_file") weightFile = v;
                else if (key == "expert_sublayer_type") sublayerType = v;
                else variant = v;
            }
        } else {
            return fail("unknown plugin field %s", key.c_str());  // reference :111-114
        }
        if (!ok) return fail("plugin field %s has the wrong type or length", key.c_str());
    }
    if (expertCount <= 0 || embeddingSize <= 0 || hiddenSize <= 0)
        return fail("expert_count, embedding_size and hidden_size are required and must be positive");
    if (!centroids || (int64_t)centroidLen != (int64_t)expertCount * embeddingSize)
        return fail("expert_centroids must hold expert_count * embedding_size = %s%ld floats", "",
                    (long)expertCount * embeddingSize);
    if (layernorm && layernormLen != embeddingSize)
        return fail("layernorm_weight must hold embedding_size = %s%ld floats", "", (long)embeddingSize);

    infmoe_layer_config cfg{};
    cfg.expert_count = expertCount;
    cfg.embedding_size = embeddingSize;
    cfg.hidden_size = hiddenSize;
    cfg.max_concurrency = maxConcurrency;
    cfg.expert_centroids = centroids;
    cfg.layernorm_weight = layernorm;
    cfg.expert_weight_file = weightFile.empty() ? nullptr : weightFile.c_str();
    cfg.expert_sublayer_type = sublayerType.c_str();
    cfg.moe_variant = variant.c_str();
    infmoe_layer* layer = nullptr;
    if (infmoe_layer_create(&cfg, &layer) != INFMOE_OK) return fail("%s", infmoe_last_error());
    auto* plugin = new MoELayerPlugin(name, layer);
    plugin->setPluginNamespace(mNamespace.c_str());
    return plugin;
}

IPluginV2* MoELayerPluginCreator::deserializePlugin(const char* name, const void* serialData,
                                                    size_t serialLength) noexcept {
    infmoe_layer* layer = nullptr;
    if (infmoe_layer_deserialize(serialData, serialLength, &layer) != INFMOE_OK)
        return fail("%s", infmoe_last_error());
    auto* plugin = new MoELayerPlugin(name, layer);
    plugin->setPluginNamespace(mNamespace.c_str());
    return plugin;
}

void MoELayerPluginCreator::setPluginNamespace(const char* pluginNamespace) noexcept {
    mNamespace = pluginNamespace ? pluginNamespace : "";
}
const char* MoELayerPluginCreator::getPluginNamespace() const noexcept { return mNamespace.c_str(); }
