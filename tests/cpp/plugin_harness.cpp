// Test harness (test infrastructure): drives include/w4_trt_plugin.h from ctypes. Compiled against
// the stand-in TensorRT header in tests/cpp/mock_trt so that the plugin / creator classes are built
// and exercised, not only the TensorRT-independent state structs.
#include <cstdio>
#include <cstring>

#include "../../include/w4_trt_plugin.h"

#ifndef W4_HAVE_TENSORRT
#error "compile with -I tests/cpp/mock_trt (or real TensorRT headers)"
#endif

using namespace w4::plugin;

namespace
{
struct Builder : nvinfer1::IExprBuilder
{
    nvinfer1::IDimensionExpr pool[64];
    int used = 0;
    nvinfer1::IDimensionExpr const* constant(int64_t v) noexcept override
    {
        pool[used].value = v;
        return &pool[used++];
    }
    nvinfer1::IDimensionExpr const* operation(nvinfer1::DimensionOperation op, nvinfer1::IDimensionExpr const& a,
        nvinfer1::IDimensionExpr const& b) noexcept override
    {
        pool[used].value = op == nvinfer1::DimensionOperation::kPROD ? a.value * b.value : a.value + b.value;
        return &pool[used++];
    }
};

nvinfer1::IPluginCreator* creator(char const* name)
{
    int32_t n = 0;
    auto* const* list = plugin_creators(n);
    for (int i = 0; i < n; ++i)
        if (!std::strcmp(list[i]->getPluginName(), name))
            return list[i];
    return nullptr;
}
} // namespace

extern "C"
{
    // Creates a plugin through its creator from plugin fields, configures it for [1, max_m] rows, runs
    // getOutputDimensions / supportsFormatCombination checks, serialises, deserialises into a second
    // object, clones that, and enqueues the clone. Returns the enqueue status, or -100 - step when one
    // of the interface checks fails. groupwise: fields (type_id, quant_algo, group_size, alpha);
    // per-channel: (type_id, weight_type_id) with quant_algo carrying weight_type_id.
    int harness_run(int groupwise, int type_id, int quant_algo, int group_size, float alpha, int max_m, int m, int n, int k,
        void const* const* inputs, int nb_inputs, void* out, void* workspace, long long workspace_size, void* stream,
        long long* workspace_wanted)
    {
        char const* name = groupwise ? kGroupwiseName : kPerChannelName;
        nvinfer1::IPluginCreator* c = creator(name);
        if (!c || std::strcmp(c->getPluginVersion(), "1") || std::strcmp(c->getPluginNamespace(), "tensorrt_llm"))
            return -101;
        nvinfer1::PluginField fields[4];
        int nf = 0;
        fields[nf++] = nvinfer1::PluginField("type_id", &type_id, nvinfer1::PluginFieldType::kINT32, 1);
        if (groupwise)
        {
            fields[nf++] = nvinfer1::PluginField("quant_algo", &quant_algo, nvinfer1::PluginFieldType::kINT32, 1);
            fields[nf++] = nvinfer1::PluginField("group_size", &group_size, nvinfer1::PluginFieldType::kINT32, 1);
            fields[nf++] = nvinfer1::PluginField("alpha", &alpha, nvinfer1::PluginFieldType::kFLOAT32, 1);
        }
        else
            fields[nf++] = nvinfer1::PluginField("weight_type_id", &quant_algo, nvinfer1::PluginFieldType::kINT32, 1);
        nvinfer1::PluginFieldCollection fc{nf, fields};
        if (c->getFieldNames()->nbFields != nf)
            return -102;
        auto* p0 = static_cast<nvinfer1::IPluginV2DynamicExt*>(c->createPlugin(name, &fc));
        if (!p0)
            return -103;
        if (std::strcmp(p0->getPluginType(), name) || p0->getNbOutputs() != 1)
            return -104;

        int const bits = groupwise ? ((quant_algo & W4_ALGO_INT8_WEIGHT) ? 8 : 4) : (quant_algo == kWeightInt4 ? 4 : 8);
        int const widx = groupwise ? ((quant_algo & W4_ALGO_PRE_QUANT_SCALE) ? 2 : 1) : 1;
        // weight extents as the network sees them
        int64_t const wcols = groupwise ? int64_t(n) * bits / 8 / 2 : int64_t(n) * bits / 8;

        // output dimensions
        Builder eb;
        nvinfer1::DimsExprs in_dims[8] = {};
        in_dims[0].nbDims = 2;
        in_dims[0].d[0] = eb.constant(m);
        in_dims[0].d[1] = eb.constant(k);
        in_dims[widx].nbDims = 2;
        in_dims[widx].d[0] = eb.constant(k);
        in_dims[widx].d[1] = eb.constant(wcols);
        nvinfer1::DimsExprs od = p0->getOutputDimensions(0, in_dims, nb_inputs, eb);
        if (od.nbDims != 2 || od.d[0]->value != m || od.d[1]->value != n)
            return -105;

        // formats
        nvinfer1::PluginTensorDesc io[8] = {};
        auto const t = static_cast<nvinfer1::DataType>(type_id);
        for (int i = 0; i <= nb_inputs; ++i)
        {
            io[i].format = nvinfer1::TensorFormat::kLINEAR;
            io[i].type = (!groupwise && i == 1) ? nvinfer1::DataType::kINT8 : t;
        }
        for (int i = 0; i <= nb_inputs; ++i)
            if (!p0->supportsFormatCombination(i, io, nb_inputs, 1))
                return -106;
        io[0].type = nvinfer1::DataType::kFLOAT;
        if (p0->supportsFormatCombination(0, io, nb_inputs, 1))
            return -107;
        io[0].type = t;
        if (p0->getOutputDataType(0, nullptr, 0) != t)
            return -108;

        // configure for the profile [1, max_m]
        nvinfer1::DynamicPluginTensorDesc din[8] = {}, dout[1] = {};
        din[0].min = nvinfer1::Dims{2, {1, k}};
        din[0].max = nvinfer1::Dims{2, {max_m, k}};
        dout[0].max = nvinfer1::Dims{2, {max_m, n}};
        p0->configurePlugin(din, nb_inputs, dout, 1);
        size_t const ws = p0->getWorkspaceSize(nullptr, 0, nullptr, 0);
        if (workspace_wanted)
            *workspace_wanted = (long long) ws;

        // serialise -> deserialise -> clone
        size_t const sz = p0->getSerializationSize();
        char blob[128];
        if (sz > sizeof(blob))
            return -109;
        p0->serialize(blob);
        auto* p1 = static_cast<nvinfer1::IPluginV2DynamicExt*>(c->deserializePlugin(name, blob, sz));
        p0->destroy();
        if (!p1 || p1->getWorkspaceSize(nullptr, 0, nullptr, 0) != ws)
            return -110;
        if (c->deserializePlugin(name, blob, sz - 1) != nullptr)
            return -111; // a truncated blob must be refused
        nvinfer1::IPluginV2DynamicExt* p2 = p1->clone();
        p1->destroy();
        if (!p2 || std::strcmp(p2->getPluginNamespace(), "tensorrt_llm"))
            return -112;

        int rc = 0;
        if (inputs)
        {
            if (ws > size_t(workspace_size))
                rc = W4_ERR_WORKSPACE;
            else
            {
                nvinfer1::PluginTensorDesc ind[8] = {};
                ind[0].dims = nvinfer1::Dims{2, {m, k}};
                ind[widx].dims = nvinfer1::Dims{2, {k, wcols}};
                void* outs[1] = {out};
                rc = p2->enqueue(ind, nullptr, inputs, outs, workspace, static_cast<cudaStream_t>(stream));
            }
        }
        p2->destroy();
        return rc;
    }

    // Creation must fail (nullptr) for configurations the library refuses.
    int harness_create_fails(int groupwise, int type_id, int quant_algo, int group_size)
    {
        char const* name = groupwise ? kGroupwiseName : kPerChannelName;
        nvinfer1::PluginField fields[3];
        fields[0] = nvinfer1::PluginField("type_id", &type_id, nvinfer1::PluginFieldType::kINT32, 1);
        fields[1] = nvinfer1::PluginField(groupwise ? "quant_algo" : "weight_type_id", &quant_algo,
            nvinfer1::PluginFieldType::kINT32, 1);
        fields[2] = nvinfer1::PluginField("group_size", &group_size, nvinfer1::PluginFieldType::kINT32, 1);
        nvinfer1::PluginFieldCollection fc{groupwise ? 3 : 2, fields};
        nvinfer1::IPluginV2* p = creator(name)->createPlugin(name, &fc);
        if (p)
        {
            p->destroy();
            return 0;
        }
        return 1;
    }

    // Input index math of the groupwise plugin: fills idx[5] = {pre_quant_scale, weight, scales, zeros, bias}.
    int harness_groupwise_indices(int quant_algo, int* idx)
    {
        GroupwiseState s;
        s.quant_algo = quant_algo;
        idx[0] = s.pre_quant_scale_idx();
        idx[1] = s.weight_idx();
        idx[2] = s.scales_idx();
        idx[3] = s.zeros_idx();
        idx[4] = s.bias_idx();
        return s.nb_inputs();
    }

    // Byte layout of the serialised state (leading fields as the reference writes them).
    int harness_serialize_groupwise(int type_id, int quant_algo, int group_size, float alpha, long long min_m, long long max_m,
        long long n, long long k, char* out, int cap)
    {
        GroupwiseState s;
        s.type_id = type_id;
        s.quant_algo = quant_algo;
        s.group_size = group_size;
        s.alpha = alpha;
        s.dims = GemmDims{min_m, max_m, n, k};
        if (cap < int(GroupwiseState::kSerializedBytes))
            return -1;
        s.serialize(out);
        return int(GroupwiseState::kSerializedBytes);
    }
}
