/*
 * C ABI of the sm_100a fused-network library (libqmlp_b200.so).
 *
 * Every entry point returns a status code (QMLP_OK == 0). On failure the message of the C++
 * exception the reference would have thrown is available from qmlp_last_error() (thread local).
 * Tensors are passed as non-owning strided views (qmlp_tensor_t), the C form of the reference's
 * qmlp::Tensor (src_cpp/include/qmlp/tensor.h:22-253). All device pointers stay owned by the
 * caller and must outlive the call; all launches go to the caller's stream and never synchronise.
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference
 * checkout).
 */
#ifndef QMLP_B200_H
#define QMLP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QMLP_API
#else
#define QMLP_API __attribute__((visibility("default")))
#endif

/* status codes; configuration_error / std::runtime_error / CKL_SAFE_CALL of src_cpp/include/qmlp/errors.h:9-90 */
enum {
    QMLP_OK = 0,
    QMLP_ERROR_RUNTIME = 1,       /* std::runtime_error (CHECK_ERROR / CHECK_DIM / CHECK_SIZE / CHECK_DTYPE) */
    QMLP_ERROR_CONFIGURATION = 2, /* qmlp::configuration_error */
    QMLP_ERROR_CUDA = 3,          /* a CUDA runtime call failed */
    QMLP_ERROR_COMPILE = 4        /* instantiating the kernel templates for a spec failed */
};

/* qmlp::Tensor::Precision, src_cpp/include/qmlp/tensor.h:25-30 */
enum { QMLP_FLOAT = 0, QMLP_HALF = 1, QMLP_DOUBLE = 2 };
/* qmlp::Tensor::Usage, src_cpp/include/qmlp/tensor.h:35-38 */
enum { QMLP_INFERENCE = 0, QMLP_GRADIENTS = 1 };
/* qmlp::FusedNetwork::AdjointMode, src_cpp/include/qmlp/fused_network.h:22-34 */
enum {
    QMLP_GRADIENTS_INPUT = 1,
    QMLP_GRADIENTS_NETWORK_WEIGHTS = 2,
    QMLP_GRADIENTS_INPUT_ENCODINGS = 4
};
/* qmlp::IEncoding::AdjointMode, src_cpp/include/qmlp/iencoding.h:113-118 */
enum { QMLP_ENCODING_INPUT_GRADIENTS = 1, QMLP_ENCODING_PARAM_GRADIENTS = 2 };

/* Non-owning strided view; strides in elements. ndim == 0 means "undefined tensor".
 * Replaces qmlp::Tensor(void*, Precision, sizes, strides), src_cpp/include/qmlp/tensor.h:72-85. */
typedef struct qmlp_tensor {
    void* data;
    int32_t precision;
    int32_t ndim;
    int64_t sizes[2];
    int64_t strides[2];
} qmlp_tensor_t;

typedef struct qmlp_network qmlp_network_t;
typedef struct qmlp_encoding qmlp_encoding_t;
typedef struct qmlp_activation qmlp_activation_t;
typedef struct qmlp_trainer qmlp_trainer_t;
typedef void* qmlp_stream_t; /* cudaStream_t / CUstream */

/* ---- library singleton: qmlp::QuickMLP, src_cpp/include/qmlp/qmlp.h:14-94 ------------------- */
QMLP_API const char* qmlp_last_error(void);
/* QuickMLP::isCudaAvailable, src_cpp/src/qmlp.cpp:41-54 */
QMLP_API int qmlp_is_cuda_available(void);
/* QuickMLP::setLogLevel(name in off|debug|info|warn|error), src_cpp/src/qmlp.cpp:56-78 */
QMLP_API int qmlp_set_log_level(const char* level);
/* QuickMLP::setCompileDebugMode / isCompileDebugMode, src_cpp/include/qmlp/qmlp.h:80-90 */
QMLP_API int qmlp_set_compile_debug_mode(int enabled);
QMLP_API int qmlp_is_compile_debug_mode(void);
/* Replaces the ckl kernel-cache directory (QuickMLP::kernelLoader, src_cpp/src/qmlp.cpp:25-39):
 * where the per-spec kernel instantiations (shared objects) are looked up and written. */
QMLP_API int qmlp_set_kernel_cache_dir(const char* dir);
QMLP_API const char* qmlp_get_kernel_cache_dir(void);
/* Directory holding the kernel template headers used to instantiate a spec. */
QMLP_API int qmlp_set_kernel_include_dir(const char* dir);

/* Kernel family used for fused inference: 0 = the best one instantiated for the spec and the batch (tcgen05 tensor-core
 * kernel when the layer widths allow it and the batch fills its tile slots, else the mma.sync kernel; a level-major
 * encoding pass in front of the tcgen05 kernel when the grid tables are much larger than L2 or when a large batch
 * (2^18 points or more) fetches 96 or more table rows per point,
 * which makes the network keep a feature buffer of up to 2^22 points and 512 MB from its first such call until it is
 * destroyed), 1 = the mma.sync kernels only, 2 = the level-major pass for every grid network, 3 = the tcgen05 kernel at
 * any batch size. Takes the place of the
 * reference's per-kernel tuning options (overwrite_blocksize_*, skew_shared_memory;
 * src_cpp/src/fused_network.cpp:45-69). */
QMLP_API int qmlp_set_kernel_path(int path);
/* Synchronises the current device and returns (then clears) its kernel status word: 0 = every kernel ran to completion;
 * bit 0 (1) = a kernel gave up on a bounded on-chip wait and its results are invalid; bits 1, 2, 3 (2, 4, 8) = a kernel
 * instantiated with bounds checks (qmlp_set_tuning("bounds_check", 1)) met a table row, a stash offset or a plane offset
 * outside the size the host declared and skipped that access. The reference has no counterpart (its
 * kernels contain no waits); debugging aids there are printf paths (src_cpp/include/qmlp/kernels/layer.cuh:28-41). */
QMLP_API int qmlp_device_status(int* status);
/* Tuning switches of the fused training step, for measurements; -1 restores the library's own choice.
 * "sort_points": copy a batch into spatial-bin order first (1; never chosen automatically: it loses on random batches); "split_scatter": table-gradient scatter as
 * its own kernel (1) or inside the backward kernel (0); "scatter_runs": 0 sends every table-gradient contribution of
 * the sorted scatter straight to the table instead of summing runs of points that share a cell first. "bounds_check": 1
 * makes networks and encodings use (and build, on first use) instantiations whose kernels test every table row, stash
 * offset and plane offset against the declared sizes, skip what lies outside and set a bit of the status word
 * (qmlp_device_status) instead of faulting - the role of the reference's debug asserts in WrappedArray
 * (src_cpp/include/qmlp/kernels/common.cuh:174-218); "bounds_shrink": n declares every size n elements smaller than it
 * is (test hook: the check fires while every access still lands in real memory). Stand in for the reference's tuning options
 * (src_cpp/src/fused_network.cpp:45-69). */
QMLP_API int qmlp_set_tuning(const char* key, int value);
/* Per-kernel device timing: while enabled, every kernel the library launches is bracketed by a CUDA event pair on its
 * stream; qmlp_read_kernel_timing waits for the recorded launches, sums them per kernel (ids: the library's kernel
 * numbers, 100 = Adam, 101 = half-copy refresh) into the caller's arrays, forgets them and returns the number of
 * distinct kernels. No counterpart in the reference (its only timing aid is the wall-clock script
 * tests_py/qmlp_tests/profile_network.py:168-188). */
QMLP_API int qmlp_set_kernel_timing(int enabled);
QMLP_API int qmlp_read_kernel_timing(int max_entries, int* kernel_ids, float* milliseconds, int* launches);

/* ---- FusedNetwork: src_cpp/include/qmlp/fused_network.h:16-340 ------------------------------- */
/* FusedNetwork::FusedNetwork(cfg, parent), src_cpp/src/fused_network.cpp:33-223. cfg is the JSON text. */
QMLP_API int qmlp_network_create(const char* cfg_json, const char* parent_dir, qmlp_network_t** out);
QMLP_API void qmlp_network_destroy(qmlp_network_t* net);
/* channelsIn/channelsOut/numLayers/numEncodings/networkParameterCount, fused_network.h:159-175 */
QMLP_API int qmlp_network_channels_in(const qmlp_network_t* net);
QMLP_API int qmlp_network_channels_out(const qmlp_network_t* net);
QMLP_API int qmlp_network_num_layers(const qmlp_network_t* net);
QMLP_API int qmlp_network_num_encodings(const qmlp_network_t* net);
QMLP_API int64_t qmlp_network_parameter_count(const qmlp_network_t* net);
/* FusedNetwork::networkParameterPrecision, src_cpp/src/fused_network.cpp:247-255 */
QMLP_API int qmlp_network_parameter_precision(const qmlp_network_t* net, int usage);
/* Padded layer geometry and offsets into the flat parameter vector: FusedNetwork::networkParameter,
 * src_cpp/src/fused_network.cpp:314-346 (weights (Cout,Cin) row-major at weights_start; bias at bias_start,
 * bias_start == -1 for a layer without bias). */
QMLP_API int qmlp_network_layer_info(const qmlp_network_t* net, int layer, int* channels_in, int* channels_out,
                                     int* use_bias, int64_t* weights_start, int64_t* bias_start);
/* FusedNetwork::encoding(idx), src_cpp/src/fused_network.cpp:235-240. The handle is owned by the network. */
QMLP_API int qmlp_network_encoding(qmlp_network_t* net, int idx, qmlp_encoding_t** out);
/* FusedNetwork::setNetworkParameter, src_cpp/src/fused_network.cpp:257-278 (1-D, exact count and dtype). */
QMLP_API int qmlp_network_set_parameter(qmlp_network_t* net, const qmlp_tensor_t* tensor, int usage);
/* FusedNetwork::initializeInferenceParameters, src_cpp/src/fused_network.cpp:280-312: U(+-1/sqrt(Cin)) over the
 * padded matrices from std::default_random_engine(seed), copied to the bound INFERENCE parameter. */
QMLP_API int qmlp_network_initialize_parameters(qmlp_network_t* net, uint64_t seed);
/* Same values written to host memory (count halfs) - lets a host-only caller build the vector. */
QMLP_API int qmlp_network_initialize_parameters_host(qmlp_network_t* net, uint64_t seed, uint16_t* dst_half);
/* FusedNetwork::inference, src_cpp/src/fused_network.cpp:507-551 */
QMLP_API int qmlp_network_inference(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                    qmlp_stream_t stream);
/* Inference from and to HOST memory. The reference has no such call: a host caller of it uploads the whole batch,
 * runs FusedNetwork::inference (src_cpp/src/fused_network.cpp:507-551) and downloads the whole result, three serial
 * steps. Here the batch is cut into chunks that move through upload -> kernel -> download on three streams, so the two
 * directions of the host link and the kernel run concurrently. host_input is (num_points, channels_in) and host_output
 * (num_points, channels_out), row-major fp32; both should be page-locked (with pageable memory the copies serialise).
 * chunk_points 0 picks a chunk of about an eighth of the batch (2^16 ... 2^20 points). The kernels run on `stream`;
 * when the call returns, everything is queued and `stream` completes after the last download. Device staging buffers
 * (3 x chunk x (channels_in + channels_out) x 4 bytes) are allocated at the first call and kept with the network. */
QMLP_API int qmlp_network_inference_host(qmlp_network_t* net, const float* host_input, float* host_output,
                                         int64_t num_points, int64_t chunk_points, qmlp_stream_t stream);
/* FusedNetwork::forwardMemory, src_cpp/src/fused_network.cpp:674-689 */
QMLP_API int qmlp_network_forward_memory(qmlp_network_t* net, int64_t num_elements, int adjoint_flags, size_t* bytes);
/* FusedNetwork::forward, src_cpp/src/fused_network.cpp:691-736 */
QMLP_API int qmlp_network_forward(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                  void* tmp_memory, qmlp_stream_t stream);
/* Forward-with-stash without any allocation, for callers that cannot call cudaMalloc (a plug-in living on a fixed
 * device-memory budget, a latency-critical loop that cannot take the synchronisation an allocation implies). It has no
 * counterpart in the reference. Same kernel, arguments and output as qmlp_network_forward; the stash goes into one
 * fixed device array of QMLP_STATIC_SCRATCH_BYTES that every GPU loading this library reserves until exit. A batch
 * whose stash (qmlp_network_forward_memory) is larger is rejected with an error. All calls on a device share that
 * array: it holds the last call's stash, and calls that overlap on the GPU race on it. The first call on a device
 * resolves the array's address (and may load the network's kernels): make it before any stream capture. */
#define QMLP_STATIC_SCRATCH_BYTES (32u << 20)
QMLP_API int qmlp_network_forward_static_scratch(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                                 qmlp_stream_t stream);
/* Device address and size of that fixed array on the current device, so that the stash the call above left there can
 * be handed on: pass the address as tmp_forward of qmlp_network_adjoint for the same batch (nothing is allocated; the
 * contents are those of the last qmlp_network_forward_static_scratch call on this device). No counterpart in the
 * reference. */
QMLP_API int qmlp_static_scratch(void** device_address, size_t* bytes);
/* FusedNetwork::zeroGradients, src_cpp/src/fused_network.cpp:738-744 (asynchronous on `stream` here). */
QMLP_API int qmlp_network_zero_gradients(qmlp_network_t* net, qmlp_stream_t stream);
/* FusedNetwork::adjointMemory, src_cpp/src/fused_network.cpp:997-1010 */
QMLP_API int qmlp_network_adjoint_memory(qmlp_network_t* net, int64_t num_elements, int adjoint_flags, size_t* bytes);
/* FusedNetwork::adjoint, src_cpp/src/fused_network.cpp:1012-1145. Gradients are accumulated (+=). */
QMLP_API int qmlp_network_adjoint(qmlp_network_t* net, const qmlp_tensor_t* input, const qmlp_tensor_t* adj_output,
                                  int adjoint_flags, qmlp_tensor_t* adj_input, const void* tmp_forward,
                                  void* tmp_adjoint, qmlp_stream_t stream);
/* FusedNetwork::clearCachedKernels, src_cpp/src/fused_network.cpp:1147-1153 */
QMLP_API int qmlp_network_clear_cached_kernels(qmlp_network_t* net);
/* Replaces the lazy compile*Kernel calls (src_cpp/src/fused_network.cpp:392-505, 553-672, 746-995): instantiate the
 * kernel templates for this spec now. Needs the compiler, not a GPU. Bit i of grid_half_mask selects the fp16-table
 * variant for the i-th grid encoding (0: all tables fp32, the reference layout). */
QMLP_API int qmlp_network_compile(qmlp_network_t* net, int grid_half_mask);
/* Number of kernel launches issued by this network object so far (for launch accounting). */
QMLP_API int64_t qmlp_network_launch_count(const qmlp_network_t* net);

/* ---- IEncoding: src_cpp/include/qmlp/iencoding.h:36-140 ------------------------------------- */
/* EncodingFactory::create, src_cpp/src/iencoding.cpp:221-228 */
QMLP_API int qmlp_encoding_create(const char* cfg_json, qmlp_encoding_t** out);
QMLP_API void qmlp_encoding_destroy(qmlp_encoding_t* enc);
/* toJson / id / maxInputChannel / numOutputChannels / hasParameters / parameterCount / parameterPrecision */
QMLP_API const char* qmlp_encoding_to_json(qmlp_encoding_t* enc);
QMLP_API const char* qmlp_encoding_id(qmlp_encoding_t* enc);
QMLP_API int qmlp_encoding_max_input_channel(const qmlp_encoding_t* enc);
QMLP_API int qmlp_encoding_num_output_channels(const qmlp_encoding_t* enc);
QMLP_API int qmlp_encoding_has_parameters(const qmlp_encoding_t* enc);
QMLP_API int64_t qmlp_encoding_parameter_count(const qmlp_encoding_t* enc);
QMLP_API int qmlp_encoding_parameter_precision(const qmlp_encoding_t* enc, int usage);
/* Level table of a grid encoding (EncodingHashGrid::getLayerConfig, src_cpp/include/qmlp/encoding_hashgrid.h:45-127,
 * computed as src_cpp/src/encoding_hashgrid.cpp:64-96). Returns the number of levels; arrays may be NULL. */
QMLP_API int qmlp_encoding_grid_levels(const qmlp_encoding_t* enc, int max_levels, int64_t* memory_offset,
                                       int32_t* resolution, int32_t* hash_grid_size, int32_t* hashed);
/* IEncoding::setParameter, src_cpp/src/encoding_hashgrid.cpp:190-202. FLOAT as in the reference; an INFERENCE
 * tensor may also be HALF (extension: fp16 gather table). An undefined tensor (ndim 0) unbinds. */
QMLP_API int qmlp_encoding_set_parameter(qmlp_encoding_t* enc, const qmlp_tensor_t* tensor, int usage);
/* IEncoding::zeroGradients, src_cpp/src/encoding_hashgrid.cpp:245-249 */
QMLP_API int qmlp_encoding_zero_gradients(qmlp_encoding_t* enc, qmlp_stream_t stream);
/* IEncoding::forward, src_cpp/src/iencoding.cpp:12-95: fp32 (B, C_in) -> fp32 (B, >= numOutputChannels).
 * `parameters` may be NULL (use the bound parameter). */
QMLP_API int qmlp_encoding_forward(qmlp_encoding_t* enc, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                   qmlp_stream_t stream, const qmlp_tensor_t* parameters);
/* IEncoding::adjoint, src_cpp/src/iencoding.cpp:97-196 */
QMLP_API int qmlp_encoding_adjoint(qmlp_encoding_t* enc, const qmlp_tensor_t* input, const qmlp_tensor_t* adj_output,
                                   qmlp_tensor_t* adj_input, qmlp_stream_t stream, const qmlp_tensor_t* parameters,
                                   qmlp_tensor_t* parameter_gradients, int adjoint_mode);

/* Instantiate the stand-alone kernels of this encoding now (replaces the lazy NVRTC compile inside IEncoding::forward,
 * src_cpp/src/iencoding.cpp:26-63). half_table selects the fp16-table variant. Needs the compiler, not a GPU. */
QMLP_API int qmlp_encoding_compile(qmlp_encoding_t* enc, int half_table);

/* ---- Activation: src_cpp/include/qmlp/activation.h:29-147 ----------------------------------- */
/* ActivationFactory::getOrInline, src_cpp/src/activation.cpp:225-240: a built-in id or an inline JSON object
 * {"id","forward","adjoint"} whose snippets are CUDA statements over `half x` -> `half z` / `half adjx`. */
QMLP_API int qmlp_activation_create(const char* key_or_json, qmlp_activation_t** out);
QMLP_API void qmlp_activation_destroy(qmlp_activation_t* act);
QMLP_API const char* qmlp_activation_id(qmlp_activation_t* act);
QMLP_API const char* qmlp_activation_to_json(qmlp_activation_t* act);
/* Activation::forward / adjoint, src_cpp/src/activation.cpp:64-150: (N, C) half tensors. */
QMLP_API int qmlp_activation_forward(qmlp_activation_t* act, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                     qmlp_stream_t stream);
QMLP_API int qmlp_activation_adjoint(qmlp_activation_t* act, const qmlp_tensor_t* input,
                                     const qmlp_tensor_t* adj_output, qmlp_tensor_t* adj_input, qmlp_stream_t stream);

/* Instantiate the stand-alone kernels of this activation now (lazy NVRTC compile in the reference,
 * src_cpp/src/activation.cpp:76-92). Needs the compiler, not a GPU. */
QMLP_API int qmlp_activation_compile(qmlp_activation_t* act);

/* ---- fused training step ---------------------------------------------------------------------
 * Not a single function in the reference: there the loss and optimiser are user PyTorch code
 * (tests_py/qmlp_tests/test_network_image.py:41-55: mse_loss + torch.optim.Adam around FusedNetwork.forward). These
 * entry points fuse that loop for one replica. All buffers are caller-owned device memory. */
typedef struct qmlp_trainer_config {
    float learning_rate, beta1, beta2, epsilon; /* torch.optim.Adam defaults of the reference demo: 1e-2, .9, .999, 1e-8 */
    int32_t grid_half_copy;                     /* 1: keep an fp16 copy of every grid table for the gather */
    int32_t reserved;
} qmlp_trainer_config_t;
QMLP_API int qmlp_trainer_create(qmlp_network_t* net, const qmlp_trainer_config_t* cfg, qmlp_trainer_t** out);
QMLP_API void qmlp_trainer_destroy(qmlp_trainer_t* tr);
/* Number of fp32 elements in the fused vector [network | encoding 0 | encoding 1 ...] and the start of each segment
 * (segment 0 = network, 1 + i = encoding i; -1 when the encoding has no parameters). */
QMLP_API int64_t qmlp_trainer_fused_count(const qmlp_trainer_t* tr);
QMLP_API int64_t qmlp_trainer_segment_start(const qmlp_trainer_t* tr, int segment);
/* Scratch bytes a step over `num_elements` points needs (stash + adjoint stash + output + output gradient). */
QMLP_API int qmlp_trainer_workspace_bytes(qmlp_trainer_t* tr, int64_t num_elements, size_t* bytes);
/* Bind the fused buffers: fp32 master parameters, fp32 gradient, Adam first/second moments (all fused_count floats)
 * and the half working copy (fused_count halfs: fp16 network weights, and fp16 grid tables when grid_half_copy). */
QMLP_API int qmlp_trainer_bind(qmlp_trainer_t* tr, float* master, float* gradient, float* adam_m, float* adam_v,
                               uint16_t* half_copy);
/* master -> half copy (call once after initialising the master parameters). */
QMLP_API int qmlp_trainer_refresh_half(qmlp_trainer_t* tr, qmlp_stream_t stream);
/* forward-with-stash, L2 loss gradient 2(out-target)/(global_points*C), backward, weight/bias/grid gradients
 * accumulated into the fused gradient buffer. loss_sum (device, 1 float, may be NULL) += sum (out-target)^2. */
QMLP_API int qmlp_trainer_gradients(qmlp_trainer_t* tr, const qmlp_tensor_t* input, const qmlp_tensor_t* target,
                                    int64_t global_points, void* workspace, size_t workspace_bytes, float* loss_sum,
                                    qmlp_stream_t stream);
/* The same step in two parts, so that a data-parallel caller can start the all-reduce of the (large) table-gradient
 * segments while the weight gradients are still being computed: parts = 1 runs forward, backward and the table-gradient
 * scatter (afterwards the encoding segments of the gradient buffer are final), parts = 2 the weight/bias gradients of
 * the layers (needs part 1 of the same batch in the same workspace), parts = 3 both. Finer still, for networks whose
 * table gradients are scattered by a kernel of their own (qmlp_trainer_scatter_levels > 0): parts = 4 runs forward and
 * backward and leaves the adjoint feature planes in the workspace; parts = 8 | first << 8 | end << 16 then scatters
 * the grid levels [first, end) (numbered over all grids as qmlp_trainer_scatter_levels lists them), after which their
 * part of the gradient buffer is final; every level must be scattered exactly once before qmlp_trainer_update. After
 * part 4 the level ranges and part 2 may follow in any order. */
QMLP_API int qmlp_trainer_gradients_part(qmlp_trainer_t* tr, const qmlp_tensor_t* input, const qmlp_tensor_t* target,
                                         int64_t global_points, void* workspace, size_t workspace_bytes,
                                         float* loss_sum, int parts, qmlp_stream_t stream);
/* Grid levels in scatter order with their element ranges [fused_begin, fused_end) in the fused buffers (arrays of
 * max_levels entries, may be NULL). Returns the number of levels, or 0 when this network's table gradients are not
 * scattered by a kernel of their own (then only parts 1, 2, 3 apply). */
QMLP_API int qmlp_trainer_scatter_levels(qmlp_trainer_t* tr, int max_levels, int64_t* fused_begin, int64_t* fused_end);
/* Adam over the fused buffer (gradient scaled by grad_scale first, e.g. 1 for a summed all-reduce of gradients
 * already normalised by global_points), refresh of the half copy, gradient buffer zeroed. step is 1-based. */
QMLP_API int qmlp_trainer_update(qmlp_trainer_t* tr, int64_t step, float grad_scale, qmlp_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QMLP_B200_H */
