/*
 * odla_b200.h -- the C ABI exported by libodla_b200.so.
 *
 * libodla_b200.so is an ODLA 0.5 platform library (a sibling of odla_dnnl and
 * odla_tensorrt in alibaba/heterogeneity-aware-lowering-and-optimization) whose
 * kernels are written for NVIDIA B200 (sm_100a).  Every type, enumerator value
 * and function signature below is binary compatible with the reference
 * headers under ODLA/include/ODLA/ so that a HALO-generated model.cc, which
 * only includes <ODLA/odla.h>, links against this library unchanged.  The
 * comment on each group names the reference header (path inside the reference
 * project, with line numbers) that the group replaces.
 *
 * The file is self contained C99 / C++11: plain pointers, sizes and PODs.
 */
#ifndef ODLA_B200_H_
#define ODLA_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar aliases: ODLA/include/ODLA/odla_common.h:56-90 ---- */
typedef __INT8_TYPE__ odla_int8;
typedef __INT16_TYPE__ odla_int16;
typedef __INT32_TYPE__ odla_int32;
typedef __INT64_TYPE__ odla_int64;
typedef __UINT8_TYPE__ odla_uint8;
typedef __UINT16_TYPE__ odla_uint16;
typedef __UINT32_TYPE__ odla_uint32;
typedef __UINT64_TYPE__ odla_uint64;
typedef __INT8_TYPE__ odla_qint8;
typedef __INT16_TYPE__ odla_qint16;
typedef __INT32_TYPE__ odla_qint32;
typedef __INT64_TYPE__ odla_qint64;
typedef __UINT8_TYPE__ odla_quint8;
typedef __UINT16_TYPE__ odla_quint16;
typedef __UINT32_TYPE__ odla_quint32;
typedef __UINT64_TYPE__ odla_quint64;
typedef __UINT16_TYPE__ odla_float16;  /* raw IEEE binary16 bits */
typedef __UINT16_TYPE__ odla_bfloat16; /* raw bfloat16 bits */
typedef float odla_float32;
typedef double odla_float64;
typedef const char* odla_string;
typedef odla_uint32 odla_bool;
typedef char odla_char;
typedef __SIZE_TYPE__ odla_size_t;
typedef void odla_void;
#ifndef NULL
#define NULL ((void*)0)
#endif
#define ODLA_API_EXPORT
#define ODLA_API_CALL

/* ---- element types: ODLA/include/ODLA/odla_common.h:99-122 ---- */
typedef enum {
  ODLA_INT8 = 0, ODLA_INT16, ODLA_INT32, ODLA_INT64,
  ODLA_UINT8, ODLA_UINT16, ODLA_UINT32, ODLA_UINT64,
  ODLA_QINT8, ODLA_QINT16, ODLA_QINT32, ODLA_QINT64,
  ODLA_QUINT8, ODLA_QUINT16, ODLA_QUINT32, ODLA_QUINT64,
  ODLA_FLOAT16, ODLA_BFLOAT16, ODLA_FLOAT32, ODLA_FLOAT64,
  ODLA_BOOL, ODLA_STRING
} odla_element_type;

/* ---- status codes: ODLA/include/ODLA/odla_common.h:140-165 ---- */
typedef enum {
  ODLA_SUCCESS = 0, ODLA_DL_ERROR, ODLA_FILE_NOT_EXIST, ODLA_INVALID_PARAM,
  ODLA_MEM_ERROR, ODLA_UNSUPPORTED_DATATYPE, ODLA_UNSUPPORTED_DEVICE_TYPE,
  ODLA_UNSUPPORTED_OP, ODLA_TIMEOUT, ODLA_INTERNAL_LOGIC_ERR,
  ODLA_RECOVERABLE_ERR, ODLA_PARTITION_RESET, ODLA_FULL_RESET,
  ODLA_UNRECOVERABLE_ERR, ODLA_FAILURE
} odla_status;

/* ---- value PODs and handles: ODLA/include/ODLA/odla_value.h:32-80 ----
 * These structs are passed BY VALUE across the ABI; their layout is fixed. */
#define ODLA_MAX_DIMENSION 10
#define ODLA_MAX_OUTPUTS 64
typedef struct {
  odla_element_type data_type;
  union {
    odla_int32 val_int32; odla_uint32 val_uint32;
    odla_int64 val_int64; odla_uint64 val_uint64;
    odla_float32 val_fp32; odla_float64 val_fp64;
    odla_string val_str;
  };
} odla_scalar_value;
typedef struct { odla_int32 size; odla_int64 dims[ODLA_MAX_DIMENSION]; } odla_value_shape;
typedef struct { odla_element_type element_type; odla_value_shape shape; } odla_value_type;
typedef struct _odla_value* odla_value;
typedef struct { odla_size_t size; odla_value values[ODLA_MAX_OUTPUTS]; } odla_values;
typedef struct _odla_value_id* odla_value_id; /* by convention a const char* name */
typedef struct { odla_size_t size; odla_value_id value_ids[ODLA_MAX_OUTPUTS]; } odla_value_ids;

/* ---- devices: ODLA/include/ODLA/odla_device.h:32-104 ---- */
typedef enum {
  ODLA_VENDOR_DEFAULT = 0, ODLA_VENDOR_ALIBABA, ODLA_VENDOR_ARM, ODLA_VENDOR_CAMBRICON,
  ODLA_VENDOR_GRAPHCORE, ODLA_VENDOR_HABANA, ODLA_VENDOR_INTEL, ODLA_VENDOR_NVIDIA,
  ODLA_VENDOR_QUALCOMM
} odla_vendor_name;
typedef enum { OVI_DESCRIPTION = 0, OVI_FEATURE_SET } odla_vendor_info;
typedef enum {
  ODLA_DEVICE_DEFAULT = 0, ODLA_DEVICE_ALIBABA_HANGUANG, ODLA_DEVICE_ARM_CORTEX_M,
  ODLA_DEVICE_CAMBRICON_MLU220, ODLA_DEVICE_CAMBRICON_MLU270, ODLA_DEVICE_GRAPHCORE_IPU,
  ODLA_DEVICE_HABANA_GAUDI, ODLA_DEVICE_HABANA_GOYA, ODLA_DEVICE_INTEL_X86,
  ODLA_DEVICE_INTEL_DNNL, ODLA_DEVICE_NVIDIA_GPU, ODLA_DEVICE_NVIDIA_TENSORRT,
  ODLA_DEVICE_QUALCOMM_AIC100
} odla_device_name;
typedef enum {
  ODLA_DEVICE_INFO_ODLA_LIB_VERSION = 0, ODLA_DEVICE_INFO_DEV_COUNT, ODLA_DEVICE_INFO_DEV_INDEX,
  ODLA_DEVICE_INFO_DEV_TYPE, ODLA_DEVICE_INFO_DEV_UUID, ODLA_DEVICE_INFO_PROCESSOR_UTIL,
  ODLA_DEVICE_INFO_MEMORY_UTIL, ODLA_DEVICE_INFO_TOTAL_MEMORY, ODLA_DEVICE_INFO_USED_MEMORY,
  ODLA_DEVICE_INFO_POWER_USAGE, ODLA_DEVICE_INFO_POWER_LIMIT, ODLA_DEVICE_INFO_DRIVER_VERSION,
  ODLA_DEVICE_INFO_SDK_VERSION
} odla_device_info;
typedef struct _odla_vendor* odla_vendor;
typedef struct _odla_device* odla_device;
typedef struct _odla_device_config* odla_device_config;
typedef struct _odla_device_config_item* odla_device_config_item;

/* ---- compute objects and property keys: ODLA/include/ODLA/odla_compute.h:33-112 ---- */
typedef enum { ODLA_COMPUTE_DEFAULT = 0, ODLA_COMPUTE_INFERENCE, ODLA_COMPUTE_TRAINING } odla_compute_mode;
typedef enum {
  ODLA_DYNAMIC_BATCH = 0, ODLA_MIN_BATCH_SIZE, ODLA_MAX_BATCH_SIZE, ODLA_OPT_BATCH_SIZE,
  ODLA_RUN_BATCH_SIZE, ODLA_DYNAMIC_SHAPE, ODLA_MIN_SHAPE, ODLA_MAX_SHAPE, ODLA_OPT_SHAPE,
  ODLA_DYNAMIC_VALUE, ODLA_MIN_VALUE, ODLA_MAX_VALUE, ODLA_OPT_VALUE, ODLA_BF16_MODE,
  ODLA_FP16_MODE, ODLA_USE_SIM_MODE, ODLA_PROCESSOR_NUM, ODLA_BATCHES_PER_STEP,
  ODLA_USE_DATA_TYPE, ODLA_LOAD_ENGINE_MODE, ODLA_USE_DLA_CORE, ODLA_QUANT_TABLE,
  ODLA_QUANT_TABLE_SIZE, ODLA_AGGREGATE_OPS, ODLA_ENABLE_ENGINE_CACHE, ODLA_CACHE_DIR,
  ODLA_ASYNC_CALLBACK_FUNC, ODLA_ASYNC_CALLBACK_ARG
} odla_item_type;
typedef enum { BF16_DISABLE = 0, BF16_ACCURACY_MODE, BF16_PERFORMACE_MODE, BF16_AUTO_MODE } odla_bf16_mode;
typedef enum { ODLA_LOCATION_PATH = 0, ODLA_LOCATION_MEMORY, ODLA_LOCATION_URI } odla_resource_location_type;
typedef struct {
  odla_resource_location_type location_type;
  const void* location;
  odla_size_t size;
} odla_resource_location;
typedef struct _odla_computation* odla_computation;
typedef struct _odla_executable* odla_executable;
typedef struct _odla_context* odla_context;
typedef struct _odla_item_value* odla_item_value;
typedef struct _odla_constants_array* odla_constants_array;

/* ---- op attribute enums: ODLA/include/ODLA/ops/odla_ops_nn.h:35-44,
 *      ODLA/include/ODLA/ops/odla_ops_process.h:33-52 ---- */
typedef enum {
  ODLA_CHANNELS_FIRST = 0, ODLA_CHANNELS_LAST, ODLA_SIO, ODLA_SOI, ODLA_OIS, ODLA_IOS
} odla_memory_layout;
typedef enum { ODLA_NEAREST = 0, ODLA_LINEAR, ODLA_CUBIC } odla_interpolation_mode;
typedef enum {
  ODLA_ASSYMMETRIC = 0, ODLA_HALF_PIXEL, ODLA_HALF_PIXEL_TF, ODLA_ALIGN_CORNERS
} odla_resize_coordinate_mode;

/* ---- quantisation table entry: ODLA/include/ODLA/ops/odla_ops_quantization.h:33-41 ---- */
typedef struct {
  odla_value_id value_id;
  int ch_idx;
  odla_float32 scale, offset, min, max;
} odla_value_quant_info;

/* ---- logging: ODLA/include/ODLA/odla_log.h:31-68 ---- */
typedef enum {
  ODLA_LOG_LEVEL_OFF = 0, ODLA_LOG_LEVEL_FATAL, ODLA_LOG_LEVEL_ERROR, ODLA_LOG_LEVEL_WARN,
  ODLA_LOG_LEVEL_INFO, ODLA_LOG_LEVEL_DEBUG, ODLA_LOG_LEVEL_TRACE
} odla_log_level;
typedef void (*odla_logging_func)(const char* file_name, int line, const char* func_name,
                                  odla_log_level level, const char* msg);
odla_status odla_SetLogLevel(odla_log_level level);
odla_status odla_SetLogger(odla_logging_func logger);
odla_logging_func odla_GetLogger();

/* ---- version: ODLA/include/ODLA/odla_version.h:29-40 ---- */
#define ODLA_MAJOR 0
#define ODLA_MINOR 5
#define ODLA_PATCH 0
const char* odla_GetVersionString();

/* ---- memory copies: ODLA/include/ODLA/odla_memory.h:32-88 ---- */
typedef enum { ODLA_MEMCPY_H2H = 0, ODLA_MEMCPY_H2D, ODLA_MEMCPY_D2H, ODLA_MEMCPY_D2D } odla_memcpy_type;
odla_status odla_AllocateDeviceMemory(odla_void** dev_ptr, odla_size_t size);
odla_status odla_FreeDeviceMemory(odla_void* ptr);
odla_status odla_AllocateHostMemory(odla_void** host_ptr, odla_size_t size); /* pinned */
odla_status odla_FreeHostMemory(odla_void* ptr);
odla_status odla_CopyMemory(odla_void* dst, odla_void* src, odla_size_t size, odla_memcpy_type type);

/* ---- device functions: ODLA/include/ODLA/odla_device.h:139-183 ---- */
odla_status odla_AllocateDevice(odla_vendor vendor, odla_device_name device_name,
                                odla_int32 device_idx, odla_device* device);
odla_status odla_GetDeviceInfo(odla_device device, odla_device_info info_type,
                               odla_scalar_value* info_value);
odla_status odla_SetCurrentDevice(odla_device device);
odla_status odla_DestroyDevice(odla_device device);

/* ---- graph life cycle, binding and execution:
 *      ODLA/include/ODLA/odla_compute.h:120-121,131-132,171-186,195-254,262-297,
 *      347-369,448-530,562-563 ---- */
odla_status odla_CreateComputation(odla_computation* computation);
odla_status odla_DestroyComputation(odla_computation computation);
odla_status odla_SetComputationItem(odla_computation computation, odla_item_type type,
                                    odla_item_value value);
/* ODLA/include/ODLA/odla_compute.h:184-186.  Hands the execute to a worker thread and returns; the context's
 * ODLA_ASYNC_CALLBACK_FUNC (int (*)(void* arg, odla_status)), if set, is called with ODLA_ASYNC_CALLBACK_ARG when
 * the outputs are written.  Bindings must stay as they are until then. */
odla_status odla_AsyncExecuteComputation(const odla_computation computation, const odla_context context,
                                         const odla_compute_mode mode, odla_device device);
/* Extension (no counterpart in the reference): waits for the context's asynchronous execute and returns its status. */
odla_status odla_b200_WaitContext(odla_context context);
/* Extension.  Contexts of one computation are spread over sets of arenas and streams ("lanes": 2 unless the environment
 * variable ODLA_B200_CONTEXT_LANES says otherwise; the second lane is built when its first context first executes).
 * Contexts on different lanes execute at the same time -- the way the reference's TensorRT platform gives each
 * odla_context an execution context and a stream of its own (ODLA/platforms/tensorrt/odla_tensorrt.h:380-394) --, contexts on the same
 * lane take turns.  Returns the lane of `context` (0, 1, ...), or -1 for a null context. */
int odla_b200_ContextLane(odla_context context);
odla_status odla_CompileComputation(const odla_computation computation, const odla_device device,
                                    odla_executable* executable);
odla_status odla_LaunchExecutable(odla_executable executable, odla_context context);
odla_status odla_DestroyExecutable(odla_executable executable);
/* ODLA/include/ODLA/odla_compute.h:347-369; shape of ODLA/platforms/tensorrt/odla_tensorrt.cc:537-559,703-811.
 * odla_StoreExecutable writes the computation behind `executable` as one self-contained file (ODLA_LOCATION_PATH):
 * the recorded graph, the constants, the computation's items and -- once it has been compiled or executed -- the
 * constants in the form the kernels read them (converted, filters repacked), so that a loaded executable plans
 * without repeating those conversions.  odla_LoadExecutable (path or memory) creates a new computation from such a
 * file, makes it the current one (odla_CreateContext attaches to it; arguments and outputs are found by id) and
 * returns it as the executable; destroy it with odla_DestroyComputation.  Nothing device-specific is stored: arenas,
 * tensor maps and CUDA graphs are rebuilt by the first execute on the GPUs the loading process sees. */
odla_status odla_LoadExecutable(odla_resource_location location, odla_device device, odla_executable* executable);
odla_status odla_StoreExecutable(odla_resource_location location, odla_executable executable);
odla_status odla_ExecuteComputation(const odla_computation computation, const odla_context context,
                                    const odla_compute_mode mode, odla_device device);
odla_status odla_GetNumOfArgsFromComputation(const odla_computation computation,
                                             odla_uint32* num_args);
odla_status odla_GetArgFromComputationByIdx(const odla_computation computation,
                                            const odla_uint32 arg_idx, odla_value* arg_value);
odla_status odla_GetNumOfOutputsFromComputation(const odla_computation computation,
                                                odla_uint32* num_outputs);
odla_status odla_GetOutputFromComputationByIdx(const odla_computation computation,
                                               const odla_uint32 output_idx,
                                               odla_value* output_value);
odla_status odla_SetValueShapeInfo(odla_value value, odla_item_type type,
                                   odla_value_shape value_shape);
odla_status odla_GetRuntimeShape(odla_context context, odla_value value,
                                 odla_value_shape* value_shape_ptr);
odla_status odla_CreateContext(odla_context* context);
odla_status odla_DestroyContext(odla_context context);
odla_status odla_SetContextItem(odla_context context, odla_item_type type, odla_item_value value);
odla_status odla_BindToArgument(odla_value value, const odla_void* data_ptr, odla_context context);
odla_status odla_BindToArgumentById(const odla_value_id value_id, const odla_void* data_ptr,
                                    odla_context context);
odla_status odla_BindToOutput(odla_value value, odla_void* data_ptr, odla_context context);
odla_status odla_BindToOutputById(const odla_value_id value_id, odla_void* data_ptr,
                                  odla_context context);

/* ---- value functions: ODLA/include/ODLA/odla_value.h:128-177 and
 *      ODLA/include/ODLA/ops/odla_ops_basic.h:39-64 ---- */
odla_value odla_CreateArgument(const odla_value_type value_type, const odla_value_id value_id);
odla_value odla_CreateConstant(const odla_value_type value_type, const odla_void* data_ptr,
                               const odla_value_id value_id);
odla_status odla_GetValueType(const odla_value value, odla_value_type* value_type);
odla_status odla_GetValueId(const odla_value value, odla_value_id* value_id);
odla_status odla_SetValueAsOutput(odla_value value);
odla_status odla_SetValuesAsOutput(odla_values values);

/* ---- neural-network ops: ODLA/include/ODLA/ops/odla_ops_nn.h:107-112 (AveragePool),
 *      172-176 (BatchNormalization), 213-219 (Conv), 274-275 (Gelu), 400-401 (LeakyRelu),
 *      413-414 (LogSoftmax), 463-467 (MaxPool), 517-518 (PRelu), 531-532 (Relu),
 *      643-644 (Sigmoid), 657-658 (Softmax) ---- */
odla_value odla_AveragePool(odla_value input, odla_memory_layout input_layout,
                            const odla_uint32* window_dims, const odla_uint32* strides,
                            const odla_uint32* paddings_front, const odla_uint32* paddings_back,
                            odla_bool padding_included, odla_value_shape output_dims,
                            const odla_value_id value_id);
odla_value odla_MaxPool(odla_value input, odla_memory_layout input_layout,
                        const odla_uint32* window_dims, const odla_uint32* strides,
                        const odla_uint32* paddings_front, const odla_uint32* paddings_back,
                        odla_value_shape output_dims, const odla_value_id value_id);
odla_value odla_BatchNormalization(odla_value input, odla_memory_layout input_layout,
                                   odla_value mean, odla_value var, odla_float32 epsilon,
                                   odla_value scale, odla_value offset, odla_float32 scalar_scale,
                                   odla_float32 scalar_offset, const odla_value_id value_id);
odla_value odla_Conv(odla_value input, odla_memory_layout input_layout, odla_uint32 group,
                     odla_value kernel, odla_memory_layout kernel_layout,
                     const odla_uint32* strides, const odla_uint32* dilations,
                     const odla_uint32* paddings_front, const odla_uint32* paddings_back,
                     odla_value bias, odla_value_shape output_dims, const odla_value_id value_id);
odla_value odla_Gelu(odla_value input, odla_bool use_approx, const odla_value_id value_id);
odla_value odla_LeakyRelu(odla_value input, odla_float32 alpha, const odla_value_id value_id);
odla_value odla_PRelu(odla_value input, odla_value slope, const odla_value_id value_id);
odla_value odla_Relu(odla_value input, const odla_value_id value_id);
odla_value odla_Sigmoid(odla_value input, const odla_value_id value_id);
odla_value odla_Softmax(odla_value input, odla_int32 axis, const odla_value_id value_id);
odla_value odla_LogSoftmax(odla_value input, odla_int32 axis, const odla_value_id value_id);

/* ---- math ops: ODLA/include/ODLA/ops/odla_ops_math.h:81-82 (Add), 234-235 (Clamp),
 *      255 (Div), 282 (Erf), 308 (Exp), 361-364 (Gemm), 337-340 (BatchMatMul), 471 (Log),
 *      538 (Mul), 551 (Neg), 616 (Pow), 630 (Reciprocal), 747-751 (ReduceMean), 817 (Round),
 *      830 (Rsqrt), 887 (Sqrt), 901 (Sub), 1004 (Tanh), 39 (Abs) ---- */
odla_value odla_Add(odla_value lhs, odla_value rhs, const odla_value_id value_id);
odla_value odla_Sub(odla_value lhs, odla_value rhs, const odla_value_id value_id);
odla_value odla_Mul(odla_value lhs, odla_value rhs, const odla_value_id value_id);
odla_value odla_Div(odla_value lhs, odla_value rhs, const odla_value_id value_id);
odla_value odla_Pow(odla_value base, odla_value exponent, const odla_value_id value_id);
odla_value odla_Abs(odla_value input, const odla_value_id value_id);
odla_value odla_Neg(odla_value input, const odla_value_id value_id);
odla_value odla_Exp(odla_value input, const odla_value_id value_id);
odla_value odla_Log(odla_value input, const odla_value_id value_id);
odla_value odla_Erf(odla_value input, const odla_value_id value_id);
odla_value odla_Sqrt(odla_value input, const odla_value_id value_id);
odla_value odla_Rsqrt(odla_value input, const odla_value_id value_id);
odla_value odla_Reciprocal(odla_value input, const odla_value_id value_id);
odla_value odla_Round(odla_value input, const odla_value_id value_id);
odla_value odla_Tanh(odla_value input, const odla_value_id value_id);
odla_value odla_Clamp(odla_value input, odla_float32 lo, odla_float32 hi,
                      const odla_value_id value_id);
odla_value odla_Gemm(odla_value A, odla_bool A_transpose, odla_value B, odla_bool B_transpose,
                     odla_float32 alpha, odla_float32 beta, odla_value C,
                     odla_value_shape output_dims, const odla_value_id value_id);
odla_value odla_BatchMatMul(odla_value A, odla_bool A_transpose, odla_value B,
                            odla_bool B_transpose, odla_value_shape output_dims,
                            const odla_value_id value_id);
odla_value odla_ReduceMean(odla_value input, odla_size_t num_of_axes, const odla_uint32* axes,
                           odla_bool keep_dims, odla_value_shape output_dims,
                           const odla_value_id value_id);

/* ---- data movement ops: ODLA/include/ODLA/ops/odla_ops_process.h:80-81 (Cast),
 *      114-115 (Concat), 168-169 (Gather), 249-250 (Reshape), 282-284 (Resize),
 *      336-338 (Slice), 434-435 (Transpose) ---- */
odla_value odla_Cast(odla_value input, odla_element_type target_type, const odla_value_id value_id);
/* ODLA/include/ODLA/ops/odla_ops_nn.h:504-507: greedy non-maximum suppression (the ONNX NonMaxSuppression rule, as
 * lib/target/generic_cpp/nms.cc emits it).  boxes [B, N, 4] (y1, x1, y2, x2), scores [B, C, N]; the result is
 * [rows, 3] int32 / int64 rows (batch, class, box) in batch, class, descending-score order, -1 where nothing is selected. */
odla_value odla_NMS(odla_value boxes, odla_value scores, odla_uint32 max_num_outputs, odla_float32 iou_threshold,
                    odla_float32 score_threshold, odla_value_type output_value_type, const odla_value_id value_id);
/* ODLA/include/ODLA/ops/odla_ops_nn.h:757-759: YOLOv3 decoding + per-class suppression of the three heads (13, 26, 52
 * cells; batch 1; NCHW or NHWC), as ODLA/platforms/odla_popart/custom_ops/postprocess.cc defines it.  Returns
 * selected_info [classes, N/169, 5] = (y_min, x_min, y_max, x_max, score) named <id>0 and selected_num [classes] named <id>1. */
odla_values odla_PostProcess(odla_value orig_img_w, odla_value orig_img_h, odla_value bb13, odla_value bb26, odla_value bb52,
                             const odla_value_id value_id);
odla_value odla_Concat(odla_values inputs, odla_int32 axis, odla_value_shape output_shape,
                       const odla_value_id value_id);
odla_value odla_Gather(odla_value input, odla_value indices, odla_int32 axis,
                       odla_value_shape output_dims, const odla_value_id value_id);
odla_value odla_Reshape(odla_value input, odla_value_shape output_dims,
                        const odla_value_id value_id);
odla_value odla_Resize(odla_value input, odla_interpolation_mode interpolation,
                       odla_resize_coordinate_mode mode, odla_uint32 axes_mask,
                       odla_value_shape output_dims, const odla_value_id value_id);
odla_value odla_Slice(odla_value input, const odla_int32* start, const odla_int32* end,
                      const odla_int32* stride, odla_value_shape output_dims,
                      const odla_value_id value_id);
odla_value odla_Transpose(odla_value input, odla_value_shape permutations,
                          odla_value_shape output_dims, const odla_value_id value_id);

/* ---- quantisation ops: ODLA/include/ODLA/ops/odla_ops_quantization.h:55-73 ---- */
odla_value odla_Dequantize(odla_value input, odla_value scale, odla_value zero_point,
                           odla_int32 axis, odla_element_type target_data_type,
                           const odla_value_id value_id);
odla_value odla_Quantize(odla_value input, odla_value scale, odla_value zero_point,
                         odla_int32 axis, odla_element_type target_data_type,
                         const odla_value_id value_id);

/* ---- LayerNorm: no ODLA header declares it, but HALO's C++ code generator emits the call
 *      when -fuse-layernorm is on (lib/target/generic_cpp/batchnorm.cc:100-113), so a
 *      platform has to define it with exactly this argument order. ---- */
odla_value odla_LayerNorm(odla_value input, odla_int32 num_of_axes, const odla_int32* axes,
                          odla_float32 epsilon, odla_value scale, odla_value offset,
                          const odla_value_id value_id);

/* =====================================================================================
 * Extensions specific to this library (no counterpart in the reference).  They never
 * change what the ODLA calls above compute; they expose placement, timing and the raw
 * kernels for tests and benchmarks.
 * ===================================================================================== */

/* Number of CUDA devices this process can see (0 without a GPU; never fails). */
int odla_b200_DeviceCount(void);

/* Binding pointers may be device pointers: odla_BindToArgument / odla_BindToOutput ask the
 * CUDA runtime what kind of memory they were given, and skip the staging copy for device
 * memory that lives on the computation's first GPU.  Nothing to call; documented here. */

/* Device time in milliseconds of the most recent odla_ExecuteComputation on `context`,
 * measured with CUDA events on the streams the kernels ran on: from the first operation
 * (the first host-to-device copy if any) to the last (the last device-to-host copy), maximum
 * over the GPUs that took part.  Returns a negative number if nothing has run. */
float odla_b200_LastExecuteDeviceMs(odla_context context);

/* Per-kernel profile of one execution.  After odla_b200_SetProfiling(context, 1), every
 * kernel launch of the next executions is bracketed by CUDA events on its stream and
 * accumulated per launch-list entry.  odla_b200_GetProfile copies up to `capacity` entries
 * (GPU 0's launch list) and returns the number of entries in the list. */
typedef struct {
  char op[32];          /* kernel family, e.g. "conv_umma", "maxpool" */
  char name[64];        /* id of the ODLA value the launch produces */
  double total_ms;      /* summed event time over the profiled executions */
  long long launches;   /* how many times it ran while profiling was on */
  double flops;         /* algorithmic 2*MAC per launch (0 for memory-bound kernels) */
  double bytes;         /* algorithmic bytes read + written per launch */
} odla_b200_profile_entry;
odla_status odla_b200_SetProfiling(odla_context context, int enabled);
int odla_b200_GetProfile(odla_context context, odla_b200_profile_entry* entries, int capacity);

/* Number of kernel launches the most recent odla_ExecuteComputation issued, all GPUs. */
long long odla_b200_LastExecuteLaunches(odla_context context);

/* Text description of the launch list (one line per kernel) into buf; returns bytes needed. */
int odla_b200_DescribePlan(odla_computation computation, char* buf, int capacity);

/* Range profiling on the GPU -- what the reference does with a wrapper platform that evaluates every op on the host and
 * records its range (ODLA/platforms/odla_profiler.cc:155-200) plus a script that turns the records into a table
 * (utils/halo_pgq.py:309-327).  While it is enabled on a context, every execute runs its launch list un-captured and
 * follows each launch by a min / max pass over the tensor it wrote (whole tensor and per channel of the last axis);
 * arguments are measured too; ranges accumulate over executes (calibration batches).  odla_b200_GetQuantTable then
 * writes the table in halo_pgq's layout -- per value one record with ch_idx = -channels, scale = max(|min|, |max|) / 127
 * and offset 0 (the symmetric int8 scheme of this library), followed by one record per channel -- ready for
 * ODLA_QUANT_TABLE.  Values that a fused kernel never writes to memory (a convolution's result before its bias and
 * ReLU) have no record; every tensor a convolution or Gemm READS has one.  Returns the number of records; call with
 * records == NULL to size the array.  The value ids point into the computation and live as long as it does. */
odla_status odla_b200_SetRangeProfiling(odla_context context, int enabled);
int odla_b200_GetQuantTable(odla_context context, odla_value_quant_info* records, int capacity);

/* How one odla_ExecuteComputation of `run_batch` rows (<= 0: the recorded batch) would be split if
 * `visible_devices` GPUs were visible: one entry per replica (GPU x sub-batch) with its device index,
 * first row and row count.  Needs no GPU -- it is the planner's shard arithmetic on its own, for
 * tests and capacity planning.  A graph whose dim 0 is not an independent batch yields one replica
 * holding every row.  Returns the number of replicas (entries beyond `capacity` are not written). */
int odla_b200_PlanShards(odla_computation computation, long long run_batch, int visible_devices,
                         int* device, long long* first_row, long long* rows, int capacity);

/* How many constants planning found already prepared (hits), had to convert itself (misses), and how many prepared
 * constants the computation holds now -- what a stored executable would carry. */
void odla_b200_PreparedConstantStats(odla_computation computation, long long* hits, long long* misses, long long* entries);

/* Raw kernel entry points over DEVICE pointers on the current device and the given stream
 * (a cudaStream_t passed as void*; NULL is the default stream).  They return 0 or a negative
 * error code (-1 bad argument, -2 CUDA error, -3 a bounded wait inside the kernel expired).
 *
 * odla_b200_conv_umma: NHWC implicit-GEMM convolution / GEMM on the tcgen05 tensor cores.
 *   x [N,H,W,C], w [K, R*S*C] (output channel major, taps then channels), y [N,P,Q,K].
 *   dtype: 0 = fp16 in/fp32 accumulate, 1 = bf16, 2 = int8 in/int32 accumulate.
 *   Epilogue: t = acc * mul[k] (mul may be NULL = 1) + add[k] (may be NULL);
 *   t += residual * res_scale (residual may be NULL); act 0 none, 1 relu, 2 leaky(alpha);
 *   out_kind 0 = same float type as input (fp16/bf16), 1 = fp32, 2 = int8 via
 *   sat(rne(t / out_scale)) -- or sat(rne(t * fl(1/out_scale))) when out_multiply is non-zero,
 *   the requantisation form the graph path uses after int32 accumulation --, 3 = raw int32
 *   accumulators (int8 input only).
 *   res_kind is the residual element type: 0 = fp16/bf16 (the input type), 1 = fp32, 2 = int8. */
typedef struct {
  int n, h, w, c, k, r, s, stride_h, stride_w, pad_top, pad_left, p, q;
  int dtype, out_kind, res_kind, act;
  float alpha, res_scale, out_scale;
  int out_multiply;
} odla_b200_conv_desc;
int odla_b200_conv_umma(const odla_b200_conv_desc* desc, const void* x, const void* w,
                        const float* mul, const float* add, const void* residual, void* y,
                        void* stream);

/* Extension (no counterpart in the reference, which leaves attention to separate MatMul / Softmax / MatMul calls:
 * lib/target/generic_cpp/matmul.cc:24-68, softmax.cc).  softmax(scale * Q K^T) V over batch * heads heads on the
 * tensor cores, the scores kept in tensor memory.  q, k, v: device pointers to [batch][heads][positions][channels] in
 * fp16 (dtype 0) or bf16 (dtype 1); only positions = 128 and channels = 64 are supported (-1 otherwise).  y is written
 * in the same layout, or as [batch][positions][heads][channels] when merge_heads is non-zero.  Synchronous on `stream`.
 * Returns 0, -1 (unsupported arguments), -2 (CUDA failure), -3 (a bounded wait inside the kernel expired).  The graph
 * path uses the same kernel when it meets this pattern (Gemm with a transposed right operand, scalar Mul, Softmax over
 * the last axis, Gemm). */
int odla_b200_attention(int dtype, const void* q, const void* k, const void* v, void* y, long long batch, int heads,
                        int positions, int channels, float scale, int merge_heads, void* stream);

/* odla_b200_reduce_mean_noalloc -- this entry point has no counterpart in the reference.
 *
 * Mean over `n_axes` axes of a dense tensor in device memory, reduced one axis after the other in
 * the order given (the arithmetic of odla_ReduceMean), without allocating anything: no cudaMalloc,
 * no cudaFree, no allocating library call.  It is for callers that cannot allocate while they run --
 * a runtime that gave all device memory to its own pool at start-up, or a serving loop that must
 * stay clear of the allocator's lock and its device-wide synchronisation.
 *
 *   x, y    device pointers on the current device; x holds prod(dims) elements, y the reduced tensor
 *   dtype   0 = fp32, 1 = fp16, 2 = bf16 (input and output)
 *   dims    extents, rank <= 10; axes: the axes to reduce, each in [0, rank) and each named once
 *           (a repeated axis, or y == x, is refused with -1: the passes do not work in place)
 *   stream  a cudaStream_t passed as void* (NULL = default stream); the kernels are only enqueued
 *
 * Intermediates between passes live in a fixed 8 MiB array inside the library image (two halves of
 * 1 Mi floats); every GPU that loads the library holds it until the process exits.  A call whose
 * intermediate after any pass but the last exceeds 1 Mi floats is refused with -1 and a message;
 * the global pool of a [N,7,7,2048] tensor fits up to N = 73.
 * The first call on a device looks up the array's device address (driver work): make that call
 * before any stream capture begins.  All calls share the array and it keeps what the last call left
 * there (nothing in it needs clearing: each pass overwrites what the next one reads), so two calls
 * whose kernels may overlap on the GPU -- different streams without an ordering between them --
 * race on it; order them.
 * Returns 0, -1 (bad argument or too large) or -2 (CUDA error). */
int odla_b200_reduce_mean_noalloc(const void* x, void* y, int dtype, const long long* dims, int rank,
                                  const int* axes, int n_axes, void* stream);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* ODLA_B200_H_ */
