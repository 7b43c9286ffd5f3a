/*
 * TensorRT plugin shim over the C ABI in w4_gemm.h: drop-in replacements for TensorRT-LLM's
 *   "WeightOnlyQuantMatmul" v1          (cpp/tensorrt_llm/plugins/weightOnlyQuantMatmulPlugin/weightOnlyQuantMatmulPlugin.cpp)
 *   "WeightOnlyGroupwiseQuantMatmul" v1 (cpp/tensorrt_llm/plugins/weightOnlyGroupwiseQuantMatmulPlugin/weightOnlyGroupwiseQuantMatmulPlugin.cpp)
 * in plugin namespace "tensorrt_llm" (tensorrt_llm/plugin/plugin.py:34), with the same plugin fields,
 * input order, output type, workspace contract and leading serialisation fields.
 *
 * Header-only, two layers:
 *   w4::plugin::*State            plain C++ (no TensorRT types): the plugin's fields, the input index
 *                                 math of init() (weightOnlyGroupwiseQuantMatmulPlugin.cpp:189-201), shape
 *                                 derivation and dispatch of enqueue (.cpp:407-495 and
 *                                 weightOnlyQuantMatmulPlugin.cpp:283-339), workspace size, serialise /
 *                                 deserialise. Always compiled; what the tests exercise.
 *   w4::plugin::*Plugin, *Creator nvinfer1::IPluginV2DynamicExt / IPluginCreator classes that forward to the
 *                                 layer above. Compiled only where <NvInferRuntime.h> is on the include
 *                                 path (TensorRT is not part of this repository's build environment).
 *
 * Differences from the reference, on purpose: no tactic profiling at engine-build time (the regime
 * choice is a pure function, w4_gemm_select_regime_typed), so the serialised tactic map is always empty
 * (count = 0) and engines are not byte-compatible with the reference's. W4A8-AWQ (FP8_ALPHA) is taken
 * for float16 plugins only, with int4 weights that the engine's emitter has re-laid
 * (w4_relayout_w4a8_to_w4a16): the scales and zeros of a W4A8 layer are float16 whatever the activation
 * type, and a plugin cannot convert engine constants in enqueue, so bfloat16 W4A8 is refused at
 * creation. enqueue never throws: it returns the negative W4Status on failure.
 */
#ifndef W4_TRT_PLUGIN_H
#define W4_TRT_PLUGIN_H

#include <cstdint>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "w4_gemm.h"

namespace w4
{
namespace plugin
{

constexpr char const* kNamespace = "tensorrt_llm";
constexpr char const* kPerChannelName = "WeightOnlyQuantMatmul";
constexpr char const* kGroupwiseName = "WeightOnlyGroupwiseQuantMatmul";
constexpr char const* kVersion = "1";

/* nvinfer1::DataType values of the type_id field. */
constexpr int kTrtHalf = 1, kTrtBf16 = 7;
/* WeightTypeId of the per-channel plugin (weightOnlyQuantMatmulPlugin.h:38-42). */
constexpr int kWeightInt8 = 1, kWeightInt4 = 2;

/* GemmDims of the reference's profiler (plugins/common/gemmPluginProfiler.h:37-60): four int64. */
struct GemmDims
{
    int64_t minM = -1, maxM = -1, n = -1, k = -1;
};

/* Shape of one tensor as the runtime hands it to enqueue (nvinfer1::Dims without the dependency). */
struct Shape
{
    int nbDims = 0;
    int64_t d[8] = {};
};

inline int act_dtype_of(int type_id)
{
    return type_id == kTrtHalf ? W4_DTYPE_FP16 : (type_id == kTrtBf16 ? W4_DTYPE_BF16 : -1);
}

inline int64_t leading_product(Shape const& s)
{
    int64_t m = 1;
    for (int i = 0; i + 1 < s.nbDims; ++i)
        m *= s.d[i];
    return m;
}

template <typename T>
inline void put(char*& p, T const& v)
{
    std::memcpy(p, &v, sizeof(T));
    p += sizeof(T);
}

template <typename T>
inline bool get(char const*& p, char const* end, T& v)
{
    if (size_t(end - p) < sizeof(T))
        return false;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return true;
}

/* ---- "WeightOnlyQuantMatmul": per-channel scales; inputs [act, weight int8 [K, N*bits/8], scales [N]] ---- */
struct PerChannelState
{
    int type_id = kTrtHalf;
    int weight_type_id = kWeightInt8;
    GemmDims dims;
    /* The plugin's weights are engine constants, so the decode kernel may fetch them ahead of the
     * preceding layer (W4_GEMM_WEIGHTS_STATIC); clear for a network that computes them on the fly. */
    bool weights_static = true;

    bool valid() const
    {
        return act_dtype_of(type_id) >= 0 && (weight_type_id == kWeightInt8 || weight_type_id == kWeightInt4);
    }

    int bits() const
    {
        return weight_type_id == kWeightInt4 ? 4 : 8;
    }

    /* n of the output from the weight tensor's second dimension (x2 for packed int4, .cpp:313). */
    int64_t real_n(Shape const& weight) const
    {
        return weight.d[1] * (weight_type_id == kWeightInt4 ? 2 : 1);
    }

    size_t workspace_bytes() const
    {
        if (dims.maxM <= 0)
            return 0;
        return w4_gemm_workspace_bytes_max(int(dims.maxM), int(dims.n), int(dims.k), 0, bits(), act_dtype_of(type_id), 0);
    }

    /* Body of enqueue: returns 0 or a negative W4Status; never throws. */
    int enqueue(Shape const& act, Shape const& weight, void const* const* inputs, void* const* outputs, void* workspace,
        size_t workspace_size, void* stream) const
    {
        if (!valid() || act.nbDims < 1 || weight.nbDims != 2)
            return W4_ERR_BAD_SHAPE;
        int64_t const m = leading_product(act);
        if (m == 0)
            return 0;
        W4GemmParams p{};
        p.act = inputs[0];
        p.weight = inputs[1];
        p.scales = inputs[2];
        p.out = outputs[0];
        p.alpha = 1.f;
        p.m = int(m);
        p.n = int(real_n(weight));
        p.k = int(act.d[act.nbDims - 1]);
        p.group_size = 0;
        p.weight_bits = bits();
        p.act_dtype = act_dtype_of(type_id);
        p.regime = W4_REGIME_AUTO;
        p.workspace = workspace;
        p.workspace_bytes = workspace_size;
        p.flags = weights_static ? W4_GEMM_WEIGHTS_STATIC : 0u;
        return w4_gemm_launch(&p, stream);
    }

    /* type, weightTypeId, GemmDims, tactic map with count = 0 (.cpp:374-391). */
    static constexpr size_t kSerializedBytes = 2 * sizeof(int32_t) + sizeof(GemmDims) + sizeof(int32_t);

    void serialize(void* buffer) const
    {
        char* p = static_cast<char*>(buffer);
        put(p, int32_t(type_id));
        put(p, int32_t(weight_type_id));
        put(p, dims);
        put(p, int32_t(0));
    }

    static bool deserialize(void const* data, size_t length, PerChannelState& out)
    {
        char const* p = static_cast<char const*>(data);
        char const* const end = p + length;
        int32_t type = 0, wtype = 0, count = 0;
        if (!get(p, end, type) || !get(p, end, wtype) || !get(p, end, out.dims) || !get(p, end, count))
            return false;
        out.type_id = type;
        out.weight_type_id = wtype;
        return out.valid(); /* a non-empty tactic map (a reference-built engine) is ignored */
    }
};

/* ---- "WeightOnlyGroupwiseQuantMatmul": inputs [act, (pre_quant_scale), weight, scales, (zeros), (bias)] ---- */
struct GroupwiseState
{
    int type_id = kTrtHalf;
    int quant_algo = 0; /* W4_ALGO_* bits */
    int group_size = 128;
    float alpha = 1.f;
    GemmDims dims;
    bool weights_static = true;

    bool valid() const
    {
        if ((quant_algo & W4_ALGO_FP8_ALPHA) && (type_id != kTrtHalf || (quant_algo & W4_ALGO_INT8_WEIGHT)))
            return false; // W4A8: float16 scales must match the activation type; int4 only
        return act_dtype_of(type_id) >= 0 && (group_size == 64 || group_size == 128);
    }

    int bits() const
    {
        return (quant_algo & W4_ALGO_INT8_WEIGHT) ? 8 : 4;
    }

    /* Input index math of the reference's init() (.cpp:197-201). */
    int pre_quant_scale_idx() const
    {
        return (quant_algo & W4_ALGO_PRE_QUANT_SCALE) ? 1 : 0;
    }
    int weight_idx() const
    {
        return pre_quant_scale_idx() + 1;
    }
    int scales_idx() const
    {
        return weight_idx() + 1;
    }
    int zeros_idx() const
    {
        return (quant_algo & W4_ALGO_ZERO) ? scales_idx() + 1 : scales_idx();
    }
    int bias_idx() const
    {
        return (quant_algo & W4_ALGO_BIAS) ? zeros_idx() + 1 : zeros_idx();
    }
    int nb_inputs() const
    {
        return bias_idx() + 1;
    }

    /* The weight arrives typed as the activation dtype, [K, N/4] (int4) or [K, N/2] (int8)
     * (.cpp:329-331, 342-355); real_n = n * 4 or n * 2 (.cpp:468). */
    int64_t real_n(Shape const& weight) const
    {
        return weight.d[1] * ((quant_algo & W4_ALGO_INT8_WEIGHT) ? 2 : 4);
    }

    size_t workspace_bytes() const
    {
        if (dims.maxM <= 0)
            return 0;
        return w4_gemm_workspace_bytes_max(int(dims.maxM), int(dims.n), int(dims.k), group_size, bits(),
            act_dtype_of(type_id), (quant_algo & W4_ALGO_PRE_QUANT_SCALE) ? 1 : 0);
    }

    int enqueue(Shape const& act, Shape const& weight, void const* const* inputs, void* const* outputs, void* workspace,
        size_t workspace_size, void* stream) const
    {
        if (!valid() || act.nbDims < 1 || weight.nbDims != 2)
            return (quant_algo & W4_ALGO_FP8_ALPHA) ? W4_ERR_UNSUPPORTED : W4_ERR_BAD_SHAPE;
        int64_t const m = leading_product(act);
        if (m == 0)
            return 0;
        W4GemmParams p{};
        p.act = inputs[0];
        p.act_scale = (quant_algo & W4_ALGO_PRE_QUANT_SCALE) ? inputs[pre_quant_scale_idx()] : nullptr;
        p.weight = inputs[weight_idx()];
        p.scales = inputs[scales_idx()];
        p.zeros = (quant_algo & W4_ALGO_ZERO) ? inputs[zeros_idx()] : nullptr;
        p.bias = (quant_algo & W4_ALGO_BIAS) ? inputs[bias_idx()] : nullptr;
        p.out = outputs[0];
        p.alpha = alpha;
        p.m = int(m);
        p.n = int(real_n(weight));
        p.k = int(act.d[act.nbDims - 1]);
        p.group_size = group_size;
        p.weight_bits = bits();
        p.act_dtype = act_dtype_of(type_id);
        p.regime = W4_REGIME_AUTO;
        p.workspace = workspace;
        p.workspace_bytes = workspace_size;
        p.flags = weights_static ? W4_GEMM_WEIGHTS_STATIC : 0u;
        return w4_gemm_launch(&p, stream);
    }

    /* type, quant_algo, group_size, alpha, GemmDims, tactic map with count = 0 (.cpp:530-551). */
    static constexpr size_t kSerializedBytes = 3 * sizeof(int32_t) + sizeof(float) + sizeof(GemmDims) + sizeof(int32_t);

    void serialize(void* buffer) const
    {
        char* p = static_cast<char*>(buffer);
        put(p, int32_t(type_id));
        put(p, int32_t(quant_algo));
        put(p, int32_t(group_size));
        put(p, alpha);
        put(p, dims);
        put(p, int32_t(0));
    }

    static bool deserialize(void const* data, size_t length, GroupwiseState& out)
    {
        char const* p = static_cast<char const*>(data);
        char const* const end = p + length;
        int32_t type = 0, algo = 0, group = 0, count = 0;
        if (!get(p, end, type) || !get(p, end, algo) || !get(p, end, group) || !get(p, end, out.alpha)
            || !get(p, end, out.dims) || !get(p, end, count))
            return false;
        out.type_id = type;
        out.quant_algo = algo;
        out.group_size = group;
        return out.valid();
    }
};

} // namespace plugin
} // namespace w4

/* ------------------------------------------------------------------------------------------------
 * TensorRT classes: only where the TensorRT headers exist.
 * ---------------------------------------------------------------------------------------------- */
#if defined(__has_include)
#if __has_include(<NvInferRuntime.h>)
#define W4_HAVE_TENSORRT 1
#include <NvInferRuntime.h>

namespace w4
{
namespace plugin
{

inline Shape shape_of(nvinfer1::Dims const& d)
{
    Shape s;
    s.nbDims = d.nbDims;
    for (int i = 0; i < d.nbDims && i < 8; ++i)
        s.d[i] = d.d[i];
    return s;
}

/* What the two plugins share: one output of the plugin's type, linear format, borrowed pointers,
 * clone = copy of the state (weightOnlyQuantMatmulPlugin.cpp:179-183), destroy = delete this (:393-397). */
template <typename Derived, typename State>
class PluginBase : public nvinfer1::IPluginV2DynamicExt
{
public:
    explicit PluginBase(State const& s)
        : mState(s)
    {
    }

    nvinfer1::IPluginV2DynamicExt* clone() const noexcept override
    {
        auto* p = new (std::nothrow) Derived(mState);
        if (p)
            p->setPluginNamespace(mNamespace.c_str());
        return p;
    }

    void configurePlugin(nvinfer1::DynamicPluginTensorDesc const* in, int32_t nbInputs,
        nvinfer1::DynamicPluginTensorDesc const* out, int32_t /*nbOutputs*/) noexcept override
    {
        /* m range from the activation's optimisation profile, n and k from the maxima
         * (weightOnlyGroupwiseQuantMatmulPlugin.cpp:357-379) */
        auto m_of = [](nvinfer1::Dims const& d)
        {
            int64_t m = 1;
            for (int i = 0; i + 1 < d.nbDims; ++i)
                m *= d.d[i];
            return m;
        };
        (void) nbInputs;
        mState.dims.minM = m_of(in[0].min);
        mState.dims.maxM = m_of(in[0].max);
        mState.dims.k = in[0].max.d[in[0].max.nbDims - 1];
        mState.dims.n = out[0].max.d[out[0].max.nbDims - 1];
    }

    size_t getWorkspaceSize(nvinfer1::PluginTensorDesc const*, int32_t, nvinfer1::PluginTensorDesc const*,
        int32_t) const noexcept override
    {
        return mState.workspace_bytes();
    }

    nvinfer1::DataType getOutputDataType(int32_t, nvinfer1::DataType const*, int32_t) const noexcept override
    {
        return static_cast<nvinfer1::DataType>(mState.type_id);
    }

    char const* getPluginVersion() const noexcept override
    {
        return kVersion;
    }
    int32_t getNbOutputs() const noexcept override
    {
        return 1;
    }
    int32_t initialize() noexcept override
    {
        return 0;
    }
    void terminate() noexcept override {}
    size_t getSerializationSize() const noexcept override
    {
        return State::kSerializedBytes;
    }
    void serialize(void* buffer) const noexcept override
    {
        mState.serialize(buffer);
    }
    void destroy() noexcept override
    {
        delete static_cast<Derived*>(this);
    }
    void setPluginNamespace(char const* ns) noexcept override
    {
        mNamespace = ns ? ns : "";
    }
    char const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }

protected:
    State mState;
    std::string mNamespace = kNamespace;
};

class WeightOnlyQuantMatmulPlugin : public PluginBase<WeightOnlyQuantMatmulPlugin, PerChannelState>
{
public:
    using PluginBase::PluginBase;

    char const* getPluginType() const noexcept override
    {
        return kPerChannelName;
    }

    nvinfer1::DimsExprs getOutputDimensions(int32_t, nvinfer1::DimsExprs const* inputs, int32_t,
        nvinfer1::IExprBuilder& eb) noexcept override
    {
        /* act [.., K] x weight [K, N or N/2] -> [.., N] (.cpp:185-227) */
        nvinfer1::DimsExprs out = inputs[0];
        auto const* n = inputs[1].d[1];
        if (mState.weight_type_id == kWeightInt4)
            n = eb.operation(nvinfer1::DimensionOperation::kPROD, *n, *eb.constant(2));
        out.d[out.nbDims - 1] = n;
        return out;
    }

    bool supportsFormatCombination(int32_t pos, nvinfer1::PluginTensorDesc const* io, int32_t, int32_t) noexcept override
    {
        /* input 1 (the weight) is int8, everything else has the plugin's type; all linear (.cpp:229-253) */
        if (io[pos].format != nvinfer1::TensorFormat::kLINEAR)
            return false;
        if (pos == 1)
            return io[pos].type == nvinfer1::DataType::kINT8;
        return io[pos].type == static_cast<nvinfer1::DataType>(mState.type_id);
    }

    int32_t enqueue(nvinfer1::PluginTensorDesc const* in, nvinfer1::PluginTensorDesc const*, void const* const* inputs,
        void* const* outputs, void* workspace, cudaStream_t stream) noexcept override
    {
        return mState.enqueue(shape_of(in[0].dims), shape_of(in[1].dims), inputs, outputs, workspace,
            mState.workspace_bytes(), stream);
    }
};

class WeightOnlyGroupwiseQuantMatmulPlugin
    : public PluginBase<WeightOnlyGroupwiseQuantMatmulPlugin, GroupwiseState>
{
public:
    using PluginBase::PluginBase;

    char const* getPluginType() const noexcept override
    {
        return kGroupwiseName;
    }

    nvinfer1::DimsExprs getOutputDimensions(int32_t, nvinfer1::DimsExprs const* inputs, int32_t,
        nvinfer1::IExprBuilder& eb) noexcept override
    {
        /* the weight is typed as the activation dtype: N = 4 x (int4) or 2 x (int8) its second extent (.cpp:290-331) */
        nvinfer1::DimsExprs out = inputs[0];
        int const factor = (mState.quant_algo & W4_ALGO_INT8_WEIGHT) ? 2 : 4;
        out.d[out.nbDims - 1] = eb.operation(nvinfer1::DimensionOperation::kPROD, *inputs[mState.weight_idx()].d[1],
            *eb.constant(factor));
        return out;
    }

    bool supportsFormatCombination(int32_t pos, nvinfer1::PluginTensorDesc const* io, int32_t, int32_t) noexcept override
    {
        /* every tensor, the weight included, carries the plugin's type (.cpp:333-355) */
        return io[pos].format == nvinfer1::TensorFormat::kLINEAR
            && io[pos].type == static_cast<nvinfer1::DataType>(mState.type_id);
    }

    int32_t enqueue(nvinfer1::PluginTensorDesc const* in, nvinfer1::PluginTensorDesc const*, void const* const* inputs,
        void* const* outputs, void* workspace, cudaStream_t stream) noexcept override
    {
        return mState.enqueue(shape_of(in[0].dims), shape_of(in[mState.weight_idx()].dims), inputs, outputs, workspace,
            mState.workspace_bytes(), stream);
    }
};

/* Creators: same field names, types and defaults as the reference's
 * (weightOnlyQuantMatmulPlugin.cpp:405-444, weightOnlyGroupwiseQuantMatmulPlugin.cpp:565-619). A bad
 * configuration yields nullptr, as the reference's creators do after catching their exception. */
template <typename Plugin, typename State>
class CreatorBase : public nvinfer1::IPluginCreator
{
public:
    char const* getPluginVersion() const noexcept override
    {
        return kVersion;
    }
    nvinfer1::PluginFieldCollection const* getFieldNames() noexcept override
    {
        mFC.nbFields = int32_t(mFields.size());
        mFC.fields = mFields.data();
        return &mFC;
    }
    nvinfer1::IPluginV2* deserializePlugin(char const*, void const* data, size_t length) noexcept override
    {
        State s;
        if (!State::deserialize(data, length, s))
            return nullptr;
        auto* p = new (std::nothrow) Plugin(s);
        if (p)
            p->setPluginNamespace(mNamespace.c_str());
        return p;
    }
    void setPluginNamespace(char const* ns) noexcept override
    {
        mNamespace = ns ? ns : "";
    }
    char const* getPluginNamespace() const noexcept override
    {
        return mNamespace.c_str();
    }

protected:
    static int32_t int_field(nvinfer1::PluginField const& f, int32_t fallback)
    {
        return f.type == nvinfer1::PluginFieldType::kINT32 && f.data ? *static_cast<int32_t const*>(f.data) : fallback;
    }
    nvinfer1::IPluginV2* make(State const& s) noexcept
    {
        if (!s.valid())
            return nullptr;
        auto* p = new (std::nothrow) Plugin(s);
        if (p)
            p->setPluginNamespace(mNamespace.c_str());
        return p;
    }
    std::vector<nvinfer1::PluginField> mFields;
    nvinfer1::PluginFieldCollection mFC{};
    std::string mNamespace = kNamespace;
};

class WeightOnlyQuantMatmulPluginCreator : public CreatorBase<WeightOnlyQuantMatmulPlugin, PerChannelState>
{
public:
    WeightOnlyQuantMatmulPluginCreator()
    {
        mFields.emplace_back("type_id", nullptr, nvinfer1::PluginFieldType::kINT32, 1);
        mFields.emplace_back("weight_type_id", nullptr, nvinfer1::PluginFieldType::kINT32, 1);
    }
    char const* getPluginName() const noexcept override
    {
        return kPerChannelName;
    }
    nvinfer1::IPluginV2* createPlugin(char const*, nvinfer1::PluginFieldCollection const* fc) noexcept override
    {
        PerChannelState s;
        for (int i = 0; i < fc->nbFields; ++i)
        {
            if (!std::strcmp(fc->fields[i].name, "type_id"))
                s.type_id = int_field(fc->fields[i], s.type_id);
            else if (!std::strcmp(fc->fields[i].name, "weight_type_id"))
                s.weight_type_id = int_field(fc->fields[i], s.weight_type_id);
        }
        return make(s);
    }
};

class WeightOnlyGroupwiseQuantMatmulPluginCreator
    : public CreatorBase<WeightOnlyGroupwiseQuantMatmulPlugin, GroupwiseState>
{
public:
    WeightOnlyGroupwiseQuantMatmulPluginCreator()
    {
        mFields.emplace_back("type_id", nullptr, nvinfer1::PluginFieldType::kINT32, 1);
        mFields.emplace_back("quant_algo", nullptr, nvinfer1::PluginFieldType::kINT32, 1);
        mFields.emplace_back("group_size", nullptr, nvinfer1::PluginFieldType::kINT32, 1);
        mFields.emplace_back("alpha", nullptr, nvinfer1::PluginFieldType::kFLOAT32, 1);
    }
    char const* getPluginName() const noexcept override
    {
        return kGroupwiseName;
    }
    nvinfer1::IPluginV2* createPlugin(char const*, nvinfer1::PluginFieldCollection const* fc) noexcept override
    {
        GroupwiseState s;
        s.quant_algo = 0;
        for (int i = 0; i < fc->nbFields; ++i)
        {
            nvinfer1::PluginField const& f = fc->fields[i];
            if (!std::strcmp(f.name, "type_id"))
                s.type_id = int_field(f, s.type_id);
            else if (!std::strcmp(f.name, "quant_algo"))
                s.quant_algo = int_field(f, s.quant_algo);
            else if (!std::strcmp(f.name, "group_size"))
                s.group_size = int_field(f, s.group_size);
            else if (!std::strcmp(f.name, "alpha") && f.type == nvinfer1::PluginFieldType::kFLOAT32 && f.data)
                s.alpha = *static_cast<float const*>(f.data);
        }
        return make(s);
    }
};

/* The two creators, for a plugin library's getPluginCreators / initLibNvInferPlugins hook
 * (cpp/tensorrt_llm/plugins/api/tllmPlugin.cpp:153, 230-232 register the reference's the same way). */
inline nvinfer1::IPluginCreator* const* plugin_creators(int32_t& count)
{
    static WeightOnlyQuantMatmulPluginCreator per_channel;
    static WeightOnlyGroupwiseQuantMatmulPluginCreator groupwise;
    static nvinfer1::IPluginCreator* const list[] = {&per_channel, &groupwise};
    count = 2;
    return list;
}

} // namespace plugin
} // namespace w4
#endif /* __has_include(<NvInferRuntime.h>) */
#endif /* defined(__has_include) */

#endif /* W4_TRT_PLUGIN_H */
