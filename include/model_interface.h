/* C ABI of a compiled model container, binary-compatible with the reference's
 * static/include/model_interface.h:41-311 (same function names, argument order, struct layouts and
 * enum values), so that the reference's ctypes binding (python/aitemplate/compiler/model.py:66-78,
 * 238-242) and its torch custom class (fx2ait/fx2ait/csrc/AITModelImpl.cpp) drive it unchanged.
 *
 * One difference: the reference links one library per model, so its Create call takes no model
 * description. This library serves every model; AITemplateModelContainerCreateFromPlan names the
 * plan file compile_model() wrote. AITemplateModelContainerCreate (no plan) reads the plan path
 * from the environment variable B200AIT_PLAN.
 */
#ifndef B200AIT_MODEL_INTERFACE_H_
#define B200AIT_MODEL_INTERFACE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#include <functional>
#include <numeric>
#define AIT_EXPORT __attribute__((__visibility__("default")))

struct AITemplateModelOpaque {};
using AITemplateModelHandle = AITemplateModelOpaque*;

enum class AITemplateError : int {
  AITemplateSuccess = 0,
  AITemplateFailure = 1,
};

struct AITemplateParamShape {
  AITemplateParamShape() : shape_data(nullptr), size(0) {}
  AITemplateParamShape(const int64_t* shape_data_in, size_t size_in) : shape_data(shape_data_in), size(size_in) {}
  const int64_t* shape_data;
  size_t size;
  size_t Numel() const {
    size_t n = 1;
    for (size_t i = 0; i < size; ++i) n *= static_cast<size_t>(shape_data[i]);
    return n;
  }
};

enum class AITemplateDtype {
  kUnset = 0,
  kHalf,
  kFloat,
  kInt,
  kLong,
  kBool,
  kBFloat16,
};

struct AITData {
  AITData() : ptr(nullptr), dtype(AITemplateDtype::kUnset) {}
  AITData(void* ptr_in, const AITemplateParamShape& shape_in, AITemplateDtype dtype_in)
      : ptr(ptr_in), shape(shape_in), dtype(dtype_in) {}
  void* ptr;
  AITemplateParamShape shape;
  AITemplateDtype dtype;
};

struct AITemplateStreamOpaque {};
using AITemplateStreamHandle = AITemplateStreamOpaque*;

/* Device allocator used for every allocation a container makes (all at creation time). */
class AITemplateAllocator {
 public:
  virtual void* Allocate(size_t nbytes) = 0;
  virtual void Free(void* ptr) = 0;
  virtual ~AITemplateAllocator() = default;
};

enum class AITemplateAllocatorType {
  kDefault = 0, /* cudaMalloc / cudaFree */
  kTracking,    /* as kDefault, and counts the bytes it handed out */
};

extern "C" {

AIT_EXPORT AITemplateError AITemplateModelContainerCreateFromPlan(AITemplateModelHandle* ret, const char* plan_path,
                                                                  size_t num_runtimes,
                                                                  AITemplateAllocator* allocator);
AIT_EXPORT AITemplateError AITemplateModelContainerCreate(AITemplateModelHandle* ret, size_t num_runtimes,
                                                          AITemplateAllocator* allocator = nullptr);
AIT_EXPORT AITemplateError AITemplateModelContainerDelete(AITemplateModelHandle handle);

AIT_EXPORT AITemplateError AITemplateModelContainerSetConstant(AITemplateModelHandle handle, const char* name,
                                                               const AITData* tensor);
AIT_EXPORT AITemplateError AITemplateModelContainerSetManyConstants(AITemplateModelHandle handle, const char** names,
                                                                    const AITData* tensors, size_t num_tensors);
AIT_EXPORT AITemplateError AITemplateModelContainerSetDoubleBufferConstant(AITemplateModelHandle handle,
                                                                           AITemplateStreamHandle stream_handle,
                                                                           const char* name, const AITData* tensor);
AIT_EXPORT AITemplateError AITemplateModelContainerSetManyDoubleBufferConstants(
    AITemplateModelHandle handle, AITemplateStreamHandle stream_handle, const char** names, const AITData* tensors,
    size_t num_tensors);
AIT_EXPORT AITemplateError AITemplateModelContainerGetNumConstants(AITemplateModelHandle handle,
                                                                   bool unbound_constants_only,
                                                                   bool constant_folding_inputs_only,
                                                                   size_t* num_constants_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetConstantNames(AITemplateModelHandle handle,
                                                                    bool unbound_constants_only,
                                                                    bool constant_folding_inputs_only,
                                                                    const char** constant_names_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetConstantDtype(AITemplateModelHandle handle, const char* name,
                                                                    AITemplateDtype* dtype);
AIT_EXPORT AITemplateError AITemplateModelContainerGetConstantOriginalName(AITemplateModelHandle handle,
                                                                           const char* name,
                                                                           const char** original_name_out);

AIT_EXPORT AITemplateError AITemplateModelContainerRun(AITemplateModelHandle handle, const AITData* inputs,
                                                       size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                       AITemplateStreamHandle stream_handle, bool sync,
                                                       bool graph_mode, int64_t** output_shapes_out);
AIT_EXPORT AITemplateError AITemplateModelContainerRunWithOutputsOnHost(
    AITemplateModelHandle handle, const AITData* inputs, size_t num_inputs, AITData* outputs, size_t num_outputs,
    AITemplateStreamHandle stream_handle, bool graph_mode, int64_t** output_shapes_out);
AIT_EXPORT AITemplateError AITemplateModelContainerProfile(AITemplateModelHandle handle, const AITData* inputs,
                                                           size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                           AITemplateStreamHandle stream_handle, size_t num_iters,
                                                           const char* filename);
AIT_EXPORT AITemplateError AITemplateModelContainerBenchmark(AITemplateModelHandle handle, const AITData* inputs,
                                                             size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                             AITemplateStreamHandle stream_handle, bool graph_mode,
                                                             size_t count, size_t num_threads,
                                                             bool use_unique_stream_per_thread, float* runtime_ms,
                                                             int64_t** output_shapes_out);

AIT_EXPORT AITemplateError AITemplateModelContainerGetNumInputs(AITemplateModelHandle handle, size_t* num_inputs_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetInputName(AITemplateModelHandle handle, size_t input_idx,
                                                                const char** input_name_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetMaximumInputShape(AITemplateModelHandle handle,
                                                                        size_t input_idx,
                                                                        AITemplateParamShape* shape);
AIT_EXPORT AITemplateError AITemplateModelContainerGetInputDtype(AITemplateModelHandle handle, size_t input_idx,
                                                                 AITemplateDtype* input_dtype);
AIT_EXPORT AITemplateError AITemplateModelContainerGetNumOutputs(AITemplateModelHandle handle,
                                                                 size_t* num_outputs_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetOutputName(AITemplateModelHandle handle, size_t output_idx,
                                                                 const char** output_name_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetMaximumOutputShape(AITemplateModelHandle handle,
                                                                         size_t output_idx,
                                                                         AITemplateParamShape* shape_out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetOutputDtype(AITemplateModelHandle handle, size_t output_idx,
                                                                  AITemplateDtype* out);
AIT_EXPORT AITemplateError AITemplateModelContainerGetNumRuntimes(AITemplateModelHandle handle,
                                                                  size_t* num_runtimes_out);

AIT_EXPORT AITemplateError AITemplateModelContainerFoldConstants(AITemplateModelHandle handle,
                                                                 AITemplateStreamHandle stream_handle, bool sync);
AIT_EXPORT AITemplateError AITemplateModelContainerFoldConstantsInDoubleBuffer(AITemplateModelHandle handle,
                                                                               AITemplateStreamHandle stream_handle,
                                                                               bool sync);
AIT_EXPORT AITemplateError AITemplateModelContainerSwapConstants(AITemplateModelHandle handle);

AIT_EXPORT AITemplateError AITemplateAllocatorCreate(AITemplateAllocator** allocator_out,
                                                     AITemplateAllocatorType allocator_type);
AIT_EXPORT AITemplateError AITemplateAllocatorDelete(AITemplateAllocator* allocator_out);
AIT_EXPORT AITemplateError AITemplateTrackingAllocatorGetNumBytes(AITemplateAllocator* allocator,
                                                                  size_t* num_bytes_out);

/* Device-memory helpers used by Model.allocate_gpu_memory / free_gpu_memory / memcpy
 * (static/include/utility.h:34-54, python/aitemplate/compiler/model.py:967-1012). */
enum class AITemplateMemcpyKind { HostToDevice = 0, DeviceToHost, DeviceToDevice };
AIT_EXPORT AITemplateError AITemplateDeviceMalloc(void** ptr_out, size_t size, AITemplateStreamHandle stream_handle,
                                                  bool sync);
AIT_EXPORT AITemplateError AITemplateDeviceFree(void* ptr, AITemplateStreamHandle stream_handle, bool sync);
AIT_EXPORT AITemplateError AITemplateMemcpy(void* dst, const void* src, size_t count, AITemplateMemcpyKind kind,
                                            AITemplateStreamHandle stream_handle, bool sync);

} /* extern "C" */
#endif /* __cplusplus */
#endif /* B200AIT_MODEL_INTERFACE_H_ */
