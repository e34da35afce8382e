// A few C entry points that play TensorRT's part towards the plugin classes -- look the creator up in
// the registry, hand it a PluginFieldCollection, call configurePlugin / getWorkspaceSize / enqueue /
// serialize / clone through the C++ virtuals -- so that the classes can be driven from tests and from
// Python without TensorRT.  Not part of the product ABI.
#include <cstring>

#include "MoELayerPlugin.h"

using namespace nvinfer1;

extern "C" {

#define TRTMOE_API __attribute__((visibility("default")))

struct trtmoe_field {
    const char* name;
    const void* data;
    int32_t type;    // nvinfer1::PluginFieldType
    int32_t length;
};

TRTMOE_API void* trtmoe_get_creator(const char* name, const char* version) {
#ifdef INFMOE_HAVE_TENSORRT
    return getPluginRegistry()->getPluginCreator(name, version, "");
#else
    return compatGetCreator(name, version);
#endif
}

TRTMOE_API int trtmoe_creator_field_names(void* creator, const char** names, int32_t max) {
    const PluginFieldCollection* fc = static_cast<IPluginCreator*>(creator)->getFieldNames();
    for (int32_t i = 0; i < fc->nbFields && i < max; ++i) names[i] = fc->fields[i].name;
    return fc->nbFields;
}

TRTMOE_API void* trtmoe_create_plugin(void* creator, const char* name, const trtmoe_field* fields, int32_t n) {
    PluginField pf[16];
    if (n > 16) return nullptr;
    for (int32_t i = 0; i < n; ++i)
        pf[i] = PluginField(fields[i].name, fields[i].data, (PluginFieldType)fields[i].type, fields[i].length);
    PluginFieldCollection fc{n, pf};
    return static_cast<IPluginCreator*>(creator)->createPlugin(name, &fc);
}

TRTMOE_API void* trtmoe_deserialize_plugin(void* creator, const char* name, const void* data, size_t len) {
    return static_cast<IPluginCreator*>(creator)->deserializePlugin(name, data, len);
}

static IPluginV2DynamicExt* P(void* p) { return static_cast<IPluginV2DynamicExt*>(static_cast<IPluginV2*>(p)); }

static PluginTensorDesc desc3(int32_t b, int32_t s, int32_t d, int32_t type, int32_t format) {
    PluginTensorDesc t{};
    t.dims.nbDims = 3;
    t.dims.d[0] = b;
    t.dims.d[1] = s;
    t.dims.d[2] = d;
    t.type = (DataType)type;
    t.format = (TensorFormat)format;
    t.scale = 1.f;
    return t;
}

TRTMOE_API const char* trtmoe_plugin_type(void* p) { return P(p)->getPluginType(); }
TRTMOE_API const char* trtmoe_plugin_version(void* p) { return P(p)->getPluginVersion(); }
TRTMOE_API int trtmoe_plugin_nb_outputs(void* p) { return P(p)->getNbOutputs(); }
TRTMOE_API int trtmoe_plugin_supports(void* p, int pos, int32_t type, int32_t format) {
    PluginTensorDesc io[2] = {desc3(1, 1, 1, type, format), desc3(1, 1, 1, type, format)};
    return P(p)->supportsFormatCombination(pos, io, 1, 1) ? 1 : 0;
}
TRTMOE_API void trtmoe_plugin_configure(void* p, int32_t b, int32_t s, int32_t d) {
    DynamicPluginTensorDesc in{}, out{};
    in.desc = out.desc = desc3(b, s, d, 0, 0);
    in.min = in.max = out.min = out.max = in.desc.dims;
    P(p)->configurePlugin(&in, 1, &out, 1);
}
TRTMOE_API size_t trtmoe_plugin_workspace(void* p, int32_t b, int32_t s, int32_t d) {
    PluginTensorDesc in = desc3(b, s, d, 0, 0), out = in;
    return P(p)->getWorkspaceSize(&in, 1, &out, 1);
}
TRTMOE_API int trtmoe_plugin_initialize(void* p) { return P(p)->initialize(); }
TRTMOE_API int trtmoe_plugin_enqueue(void* p, int32_t b, int32_t s, int32_t d, const void* in, void* out, void* ws,
                                     void* stream) {
    PluginTensorDesc din = desc3(b, s, d, 0, 0), dout = din;
    const void* ins[1] = {in};
    void* outs[1] = {out};
    return P(p)->enqueue(&din, &dout, ins, outs, ws, (cudaStream_t)stream);
}
TRTMOE_API size_t trtmoe_plugin_serialization_size(void* p) { return P(p)->getSerializationSize(); }
TRTMOE_API void trtmoe_plugin_serialize(void* p, void* buf) { P(p)->serialize(buf); }
TRTMOE_API void* trtmoe_plugin_clone(void* p) { return static_cast<IPluginV2*>(P(p)->clone()); }
TRTMOE_API void trtmoe_plugin_set_namespace(void* p, const char* ns) { P(p)->setPluginNamespace(ns); }
TRTMOE_API const char* trtmoe_plugin_namespace(void* p) { return P(p)->getPluginNamespace(); }
TRTMOE_API void* trtmoe_plugin_layer(void* p) { return static_cast<MoELayerPlugin*>(P(p))->layer(); }
TRTMOE_API void trtmoe_plugin_delete(void* p) {
    P(p)->terminate();
    P(p)->destroy();
    delete P(p);
}

}  // extern "C"
