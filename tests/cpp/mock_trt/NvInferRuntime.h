// Test stand-in for TensorRT's <NvInferRuntime.h> (test infrastructure, NOT TensorRT): just enough
// of the nvinfer1 plugin interfaces, with their public signatures, for include/w4_trt_plugin.h to be
// compiled and its plugin / creator classes to be driven from a test on a machine without
// TensorRT. Nothing here implements TensorRT behaviour.
#pragma once
#include <cstddef>
#include <cstdint>

typedef struct CUstream_st* cudaStream_t;

namespace nvinfer1
{
enum class DataType : int32_t { kFLOAT = 0, kHALF = 1, kINT8 = 2, kINT32 = 3, kBOOL = 4, kUINT8 = 5, kFP8 = 6, kBF16 = 7 };
enum class TensorFormat : int32_t { kLINEAR = 0 };
enum class PluginFieldType : int32_t { kFLOAT16 = 0, kFLOAT32 = 1, kFLOAT64 = 2, kINT8 = 3, kINT16 = 4, kINT32 = 5 };
enum class DimensionOperation : int32_t { kSUM = 0, kPROD = 1 };

struct Dims { int32_t nbDims; int64_t d[8]; };
struct PluginTensorDesc { Dims dims; DataType type; TensorFormat format; float scale; };
struct DynamicPluginTensorDesc { PluginTensorDesc desc; Dims min; Dims max; Dims opt; };

class IDimensionExpr { public: int64_t value = 0; };
struct DimsExprs { int32_t nbDims; IDimensionExpr const* d[8]; };
class IExprBuilder
{
public:
    virtual IDimensionExpr const* constant(int64_t value) noexcept = 0;
    virtual IDimensionExpr const* operation(DimensionOperation op, IDimensionExpr const& a, IDimensionExpr const& b) noexcept = 0;
    virtual ~IExprBuilder() = default;
};

struct PluginField
{
    char const* name; void const* data; PluginFieldType type; int32_t length;
    PluginField(char const* n = nullptr, void const* d = nullptr, PluginFieldType t = PluginFieldType::kFLOAT32, int32_t l = 0)
        : name(n), data(d), type(t), length(l) {}
};
struct PluginFieldCollection { int32_t nbFields; PluginField const* fields; };

class IPluginV2
{
public:
    virtual char const* getPluginType() const noexcept = 0;
    virtual char const* getPluginVersion() const noexcept = 0;
    virtual int32_t getNbOutputs() const noexcept = 0;
    virtual int32_t initialize() noexcept = 0;
    virtual void terminate() noexcept = 0;
    virtual size_t getSerializationSize() const noexcept = 0;
    virtual void serialize(void* buffer) const noexcept = 0;
    virtual void destroy() noexcept = 0;
    virtual void setPluginNamespace(char const* ns) noexcept = 0;
    virtual char const* getPluginNamespace() const noexcept = 0;
    virtual ~IPluginV2() = default;
};
class IPluginV2Ext : public IPluginV2
{
public:
    virtual DataType getOutputDataType(int32_t index, DataType const* inputTypes, int32_t nbInputs) const noexcept = 0;
};
class IPluginV2DynamicExt : public IPluginV2Ext
{
public:
    virtual IPluginV2DynamicExt* clone() const noexcept = 0;
    virtual DimsExprs getOutputDimensions(int32_t outputIndex, DimsExprs const* inputs, int32_t nbInputs, IExprBuilder& exprBuilder) noexcept = 0;
    virtual bool supportsFormatCombination(int32_t pos, PluginTensorDesc const* inOut, int32_t nbInputs, int32_t nbOutputs) noexcept = 0;
    virtual void configurePlugin(DynamicPluginTensorDesc const* in, int32_t nbInputs, DynamicPluginTensorDesc const* out, int32_t nbOutputs) noexcept = 0;
    virtual size_t getWorkspaceSize(PluginTensorDesc const* inputs, int32_t nbInputs, PluginTensorDesc const* outputs, int32_t nbOutputs) const noexcept = 0;
    virtual int32_t enqueue(PluginTensorDesc const* inputDesc, PluginTensorDesc const* outputDesc, void const* const* inputs, void* const* outputs, void* workspace, cudaStream_t stream) noexcept = 0;
};
class IPluginCreator
{
public:
    virtual char const* getPluginName() const noexcept = 0;
    virtual char const* getPluginVersion() const noexcept = 0;
    virtual PluginFieldCollection const* getFieldNames() noexcept = 0;
    virtual IPluginV2* createPlugin(char const* name, PluginFieldCollection const* fc) noexcept = 0;
    virtual IPluginV2* deserializePlugin(char const* name, void const* serialData, size_t serialLength) noexcept = 0;
    virtual void setPluginNamespace(char const* ns) noexcept = 0;
    virtual char const* getPluginNamespace() const noexcept = 0;
    virtual ~IPluginCreator() = default;
};
} // namespace nvinfer1
