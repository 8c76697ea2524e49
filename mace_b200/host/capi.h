/*
 * C entry points of the C++ host layer (libmace_b200_host.so), so that the
 * operators, delegators and the sequential net can be driven from tests and
 * benchmarks written in another language.  An engine owns one CudaRuntime, a
 * workspace of named tensors, the delegator and operator registries and a
 * SerialNet -- the roles of SerialEngine / CpuRefFlow / SerialNet in the
 * reference (mace/libmace/engines/serial_engine.cc:57-113,
 * mace/flows/cpu/cpu_ref_flow.cc:32-79, mace/core/net/serial_net.cc:93-228).
 * Every function returns a MaceStatus::Code integer.
 */
#ifndef MACE_B200_HOST_CAPI_H_
#define MACE_B200_HOST_CAPI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mbh_engine mbh_engine;

int mbh_engine_create(int device, mbh_engine **engine);
int mbh_engine_destroy(mbh_engine *engine);
const char *mbh_last_error(const mbh_engine *engine);
/* The mb_context of the engine's runtime (for event timing / launch counts). */
void *mbh_engine_context(mbh_engine *engine);

/* Creates (or replaces) a named tensor; data_type is a mace DataType value
 * (1 float, 2 uint8, 4 int32).  host_data may be NULL (uninitialised). */
int mbh_add_tensor(mbh_engine *engine, const char *name, int data_type, int rank,
                   const int64_t *dims, const void *host_data, float scale,
                   int32_t zero_point, int is_weight);
int mbh_set_tensor_quant(mbh_engine *engine, const char *name, float scale, int32_t zero_point);
int mbh_tensor_rank(mbh_engine *engine, const char *name, int *rank);
int mbh_tensor_shape(mbh_engine *engine, const char *name, int64_t *dims, int max_rank);
int mbh_tensor_quant(mbh_engine *engine, const char *name, float *scale, int32_t *zero_point);
/* Synchronous copies between a tensor and host memory. */
int mbh_tensor_read(mbh_engine *engine, const char *name, void *host_out, size_t bytes);
int mbh_tensor_write(mbh_engine *engine, const char *name, const void *host_in, size_t bytes);
/* The tensor's device address and size after the last run (Tensor::memory<T>(),
 * mace/core/memory/buffer.h:41-59), for a caller that hands it to another library on the same
 * stream -- the final gather of the output rows, for one.  Valid until the tensor is resized. */
int mbh_tensor_device_ptr(mbh_engine *engine, const char *name, void **device_ptr, size_t *bytes);

/* Operator construction, the fields of an OperatorDef (mace/proto/mace.proto:61-95). */
int mbh_op_begin(mbh_engine *engine, const char *type, const char *name);
int mbh_op_input(mbh_engine *engine, const char *tensor_name);
/* data_type < 0: take it from the op's "T" argument; scale <= 0: no quantize_info. */
int mbh_op_output(mbh_engine *engine, const char *tensor_name, int data_type, float scale,
                  int32_t zero_point);
int mbh_op_arg_int(mbh_engine *engine, const char *key, int value);
int mbh_op_arg_ints(mbh_engine *engine, const char *key, int count, const int *values);
int mbh_op_arg_floats(mbh_engine *engine, const char *key, int count, const float *values);
int mbh_op_arg_float(mbh_engine *engine, const char *key, float value);
int mbh_op_arg_str(mbh_engine *engine, const char *key, const char *value);
int mbh_op_end(mbh_engine *engine);

/* Merges each Activation operator into the operator producing its input where that operator
 * can apply the activation itself (the float Eltwise) and nothing else reads the tensor in
 * between, which is then no longer written.  *merged (may be NULL) receives the number of
 * merged pairs. */
int mbh_fuse_activations(mbh_engine *engine, int *merged);

/* After one run and after mbh_fuse_activations: merges each element-wise SUM of two tensors
 * (with the activation it has absorbed) into the float Conv2D that produces one of them, when
 * nothing else reads that tensor and the other one exists before the convolution runs: the
 * convolution then writes activation(conv + residual) into the sum's output. */
int mbh_fuse_residual_sums(mbh_engine *engine, int *merged);

/* Where several strided 1x1 float convolutions read one tensor with the same strides, gathers
 * the pixels they read once (a Subsample operator in front of the first) and runs them as
 * stride-1 convolutions of that copy.  Call before the first run or before the merging passes
 * above.  *groups (may be NULL) receives the number of shared gathers. */
int mbh_share_subsampled_inputs(mbh_engine *engine, int *groups);

/* Shares activation memory between tensors whose lifetimes do not overlap (MACE's SERIAL_OPT
 * allocation strategy).  Call after one run; intermediate tensors cannot be read back afterwards.
 * The two sizes (may be NULL) are the activation bytes before and after. */
int mbh_plan_memory(mbh_engine *engine, size_t *separate_bytes, size_t *shared_bytes);

/* The same as mbh_run_host without waiting: the upload of this call's input (from PINNED host
 * memory, on the runtime's upload stream, straight into the input tensor) starts as soon as the
 * previous call's net has passed the last operator that reads that tensor (the net records an
 * event there; a captured net is replayed as two graphs around it) and overlaps the rest of the
 * previous run.  *slot (0 or 1, may be NULL) names the call for mbh_wait_slot, which blocks until
 * that call's output is in host_out; host_in and host_out must stay untouched until then, so
 * rotate at least two host buffers of each.  Run the net once the ordinary way first.  Use one
 * input name per engine between plain runs (a plain mbh_run_host in between is fine). */
int mbh_run_host_pipelined(mbh_engine *engine, const char *input_name, const void *host_in, size_t input_bytes,
                           const char *output_name, void *host_out, size_t output_bytes, int *slot);
int mbh_wait_slot(mbh_engine *engine, int slot);

/* Runs all operators once (asynchronously on the engine's stream). */
int mbh_run(mbh_engine *engine);
int mbh_sync(mbh_engine *engine);
/* Records the operator chain into a CUDA graph that later mbh_run / mbh_run_host calls
 * replay (SerialNet::Capture).  Needs one plain mbh_run first; adding an operator or
 * replacing a tensor drops the recording. */
int mbh_capture(mbh_engine *engine);
/* Host-buffer run, the shape of MaceEngine::Run (mace/libmace/mace_engine.cc:203-212):
 * copies input_bytes from pinned or pageable host memory into the input
 * tensor, runs the net, copies the output tensor back and waits. */
int mbh_run_host(mbh_engine *engine, const char *input_name, const void *host_in,
                 size_t input_bytes, const char *output_name, void *host_out,
                 size_t output_bytes);
/* Per-operator device times of one run; returns the operator count.  names_out
 * receives "type:name" strings separated by newlines. */
int mbh_run_profiled(mbh_engine *engine, float *ms_out, int max_ops, char *names_out,
                     size_t names_len, int *op_count);

/* The same inside a graph replay (SerialNet::RunProfiledGraph): the operators are recorded into
 * a graph with an event node behind each and the graph is replayed `replays` times; the times
 * add up to the graph's duration. */
int mbh_run_profiled_graph(mbh_engine *engine, int replays, float *ms_out, int max_ops, char *names_out,
                           size_t names_len, int *op_count);

/* ---- Model files: the serialized NetDef of a converted model (mace/proto/mace.proto) and its
 * weights blob, loaded and run the way CreateMaceEngineFromProto / MaceEngine::Run do
 * (include/mace/public/mace.h:553-655). ---- */

/* Parses a serialized NetDef and writes a JSON rendering of every field into json_out (always
 * NUL-terminated, truncated to capacity); *needed (may be NULL) receives the full length
 * including the terminator.  Needs no GPU.  MACE_INVALID_ARGS for a malformed message, with
 * the reason in json_out. */
int mbh_netdef_describe(const void *graph, size_t graph_len, char *json_out, size_t capacity, size_t *needed);

/* The widening applied to DT_HALF weights when a model is loaded (IEEE binary16 -> binary32,
 * subnormals, infinities and NaN payloads included).  Needs no GPU. */
int mbh_half_to_float(const uint16_t *in, float *out, size_t count);

typedef struct mbh_model mbh_model;

/* One input or output in host memory, the fields of a MaceTensor: data_format 0 none, 1 NHWC,
 * 2 NCHW; data_type 1 float, 2 uint8, 4 int32.  For an output, shape/rank state the buffer's
 * capacity going in and the actual shape coming out. */
typedef struct mbh_io_tensor {
  const char *name;
  void *data;
  int64_t shape[8];
  int rank;
  int data_format;
  int data_type;
} mbh_io_tensor;

/* fuse / plan_memory / cuda_graph: the MaceEngineConfig switches of this runtime (merge
 * activations and residual sums, share activation memory, replay a CUDA graph), applied after
 * the first run.  On failure the reason is copied into error (may be NULL). */
int mbh_model_create(int device, const void *graph, size_t graph_len, const void *weights, size_t weights_len,
                     int fuse, int plan_memory, int cuda_graph, mbh_model **model, char *error, size_t error_len);
int mbh_model_destroy(mbh_model *model);
const char *mbh_model_last_error(const mbh_model *model);
void *mbh_model_context(mbh_model *model);
/* 1 when the operator chain is currently recorded in a CUDA graph. */
int mbh_model_captured(mbh_model *model);
int mbh_model_run(mbh_model *model, int n_inputs, const mbh_io_tensor *inputs, int n_outputs,
                  mbh_io_tensor *outputs);

/* ---- Several GPUs: one engine, stream and host thread per shard (MultiGpuRunner); the batch
 * (first dimension of every input and output) is split into contiguous shards, each shard's
 * output rows are copied device-to-host straight into its slice of the caller's buffer.  The
 * reference runs one net on one device (mace/core/net/serial_net.cc:103-124) and allows several
 * engines in parallel threads (test/ccunit/mace/libmace/mace_api_mt_test.cc:100-110). ---- */

/* Shard `index` of `parts` over `total` items (contiguous, the first total % parts shards one
 * longer).  Needs no GPU. */
int mbh_shard_bounds(int64_t total, int parts, int index, int64_t *begin, int64_t *end);

typedef struct mbh_multi mbh_multi;

/* devices[i]: CUDA ordinal of shard i (ordinals may repeat).  The other arguments as for
 * mbh_model_create. */
int mbh_multi_create(int n_shards, const int *devices, const void *graph, size_t graph_len, const void *weights,
                     size_t weights_len, int fuse, int plan_memory, int cuda_graph, mbh_multi **runner, char *error,
                     size_t error_len);
int mbh_multi_destroy(mbh_multi *runner);
const char *mbh_multi_last_error(const mbh_multi *runner);
int mbh_multi_shards(const mbh_multi *runner);
/* As mbh_model_run, on the whole batch. */
int mbh_multi_run(mbh_multi *runner, int n_inputs, const mbh_io_tensor *inputs, int n_outputs,
                  mbh_io_tensor *outputs);

/* ---- Logging (MACE_CPP_MIN_LOG_LEVEL, MACE_CPP_MIN_VLOG_LEVEL: include/mace/port/logger.h:40-58).
 * Lines go to stderr unless a sink is installed (NULL restores stderr); the sink is called from
 * whichever thread logs.  mbh_set_vlog_level overrides the environment's VLOG level
 * (INT_MIN: back to the environment).  mbh_log writes one line at `severity` (1 INFO, 2 WARNING,
 * 3 ERROR) through the same path; mbh_vlog_is_on answers what VLOG(level) would do.  No GPU
 * needed. ---- */
typedef void (*mbh_log_sink)(int severity, const char *line);
int mbh_set_log_sink(mbh_log_sink sink);
int mbh_set_vlog_level(int level);
int mbh_vlog_is_on(int level);
int mbh_log(int severity, const char *message);

/* Per-operator statistics of one run of a model (RunMetadata, include/mace/public/mace.h:177-201)
 * as JSON: [{"name":..,"type":..,"device_ms":..,"start_micros":..,"end_micros":..,
 * "output_shape":[[..]],"strides":[..],"padding_type":..,"paddings":[..],"dilations":[..],
 * "kernels":[..]}, ...].  The inputs already on the device from the last mbh_model_run are
 * used.  json_out is always NUL-terminated; *needed (may be NULL) receives the full length. */
int mbh_model_run_metadata(mbh_model *model, char *json_out, size_t capacity, size_t *needed);

#ifdef __cplusplus
}
#endif

#endif /* MACE_B200_HOST_CAPI_H_ */
