/* ggml_base_b200.h — the libggml-base-shaped export set of libggml-b200.so.
 *
 * The reference's ForeignExecutor does not talk to a backend's vtables: it dlopens a ggml build, resolves the
 * 55 symbols of CLibSyms by name (crates/ggml/src/sysffi.rs:458-629) and drives them in the order of
 * ggml-backend.h's example flow (crates/ggml/src/backend_emit.rs:439-572 new, :895-1042 graph_compute):
 *   load_all_from_path, dev_by_type(CPU) / dev_by_name, dev_init, sched_new([gpu, cpu]), ggml_init (metadata
 *   contexts), buft_alloc_buffer + tensor_alloc + tensor_set (weights, KV), and per step: ggml_init, new_tensor
 *   + direct writes of op / src / op_params / nb, build_forward_expand, sched_alloc_graph, tensor_set (inputs),
 *   sched_graph_compute, sched_synchronize, tensor_get, sched_reset.
 * This header declares those symbols with the C signatures sysffi.rs:262-347 binds, over the vtables of
 * ggml_b200_backend.h, so that pointing the executor's lib_dir at this library drives the B200 backend with
 * no change on the reference's side.
 *
 * What is behind them: a metadata-only ggml context (an arena of ggml_tensor structs), the graph builder
 * (depth-first, sources before users, each tensor once), a registry of the CUDA devices plus one "CPU" device
 * that owns host buffers but computes nothing, and a one-device scheduler: every node of a graph runs on the
 * B200 backend (alloc_graph refuses a graph with a node supports_op rejects — there is no CPU compute path),
 * step tensors live in one device compute buffer, and a source that sits in a host buffer (a weight a
 * partial -ngl placement left on the CPU side) is mirrored to the device before the compute, once for
 * buffers whose usage is WEIGHTS.
 */
#ifndef GGML_BASE_B200_H
#define GGML_BASE_B200_H

#include "ggml_b200_backend.h"

#ifdef __cplusplus
extern "C" {
#endif

struct ggml_context;
typedef struct ggml_backend_sched *ggml_backend_sched_t;

/* struct ggml_init_params (sysffi.rs:229-235); only metadata contexts are served: tensors get their data
 * from buffers (no_alloc = true is what the executor passes; with no_alloc = false data follows the struct) */
struct ggml_init_params {
    size_t mem_size;
    void *mem_buffer;
    bool no_alloc;
};

enum { GGML_TENSOR_FLAG_INPUT = 1, GGML_TENSOR_FLAG_OUTPUT = 2, GGML_TENSOR_FLAG_PARAM = 4 };
/* enum ggml_status as the reference binds it (sysffi.rs:359-363) */
enum { GGML_STATUS_SUCCESS = 0, GGML_STATUS_ALLOC_FAILED = 1, GGML_STATUS_BACKEND_ERROR = 3, GGML_STATUS_ABORTED = 4 };

/* ---- core (sysffi.rs:241-253) ---- */
struct ggml_context *ggml_init(struct ggml_init_params params);
void ggml_free(struct ggml_context *ctx);
struct ggml_tensor *ggml_new_tensor(struct ggml_context *ctx, int type, int n_dims, const int64_t *ne);
struct ggml_tensor *ggml_set_name(struct ggml_tensor *tensor, const char *name);
void ggml_set_input(struct ggml_tensor *tensor);
void ggml_set_output(struct ggml_tensor *tensor);
size_t ggml_tensor_overhead(void);
size_t ggml_graph_overhead_custom(size_t size, bool grads);
struct ggml_cgraph *ggml_new_graph_custom(struct ggml_context *ctx, size_t size, bool grads);
void ggml_build_forward_expand(struct ggml_cgraph *cgraph, struct ggml_tensor *tensor);
int ggml_graph_n_nodes(struct ggml_cgraph *cgraph);
struct ggml_tensor *ggml_graph_node(struct ggml_cgraph *cgraph, int i);   /* i < 0 counts from the end */
struct ggml_tensor **ggml_graph_nodes(struct ggml_cgraph *cgraph);

/* ---- buffers / transport (sysffi.rs:255-279) ---- */
ggml_backend_buffer_t ggml_backend_buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size);
size_t ggml_backend_buft_get_alignment(ggml_backend_buffer_type_t buft);
size_t ggml_backend_buft_get_max_size(ggml_backend_buffer_type_t buft);
size_t ggml_backend_buft_get_alloc_size(ggml_backend_buffer_type_t buft, const struct ggml_tensor *tensor);
void ggml_backend_buffer_free(ggml_backend_buffer_t buffer);
void *ggml_backend_buffer_get_base(ggml_backend_buffer_t buffer);
void ggml_backend_buffer_clear(ggml_backend_buffer_t buffer, uint8_t value);
void ggml_backend_buffer_set_usage(ggml_backend_buffer_t buffer, int usage);
void ggml_backend_tensor_set(struct ggml_tensor *tensor, const void *data, size_t offset, size_t size);
void ggml_backend_tensor_get(const struct ggml_tensor *tensor, void *data, size_t offset, size_t size);
int ggml_backend_tensor_alloc(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor, void *addr);
int ggml_backend_view_init(struct ggml_tensor *tensor);
ggml_backend_buffer_t ggml_backend_cpu_buffer_from_ptr(void *ptr, size_t size);
ggml_backend_buffer_type_t ggml_backend_cpu_buffer_type(void);

/* ---- devices / registry (sysffi.rs:281-296) ---- */
size_t ggml_backend_dev_count(void);
ggml_backend_dev_t ggml_backend_dev_get(size_t index);
ggml_backend_dev_t ggml_backend_dev_by_name(const char *name);
ggml_backend_dev_t ggml_backend_dev_by_type(int type);
const char *ggml_backend_dev_name(ggml_backend_dev_t device);
void ggml_backend_free(ggml_backend_t backend);
ggml_backend_t ggml_backend_dev_init(ggml_backend_dev_t device, const char *params);
ggml_backend_buffer_type_t ggml_backend_dev_buffer_type(ggml_backend_dev_t device);
ggml_backend_reg_t ggml_backend_dev_backend_reg(ggml_backend_dev_t device);
void *ggml_backend_reg_get_proc_address(ggml_backend_reg_t reg, const char *name);
void ggml_backend_load_all_from_path(const char *dir_path);   /* the B200 backend is built in: nothing to load */

/* ---- scheduler (sysffi.rs:298-347) ---- */
ggml_backend_sched_t ggml_backend_sched_new(ggml_backend_t *backends, ggml_backend_buffer_type_t *bufts, int n_backends,
                                            size_t graph_size, bool parallel, bool op_offload);
void ggml_backend_sched_free(ggml_backend_sched_t sched);
void ggml_backend_sched_reset(ggml_backend_sched_t sched);
bool ggml_backend_sched_alloc_graph(ggml_backend_sched_t sched, struct ggml_cgraph *graph);
int ggml_backend_sched_graph_compute(ggml_backend_sched_t sched, struct ggml_cgraph *graph);
void ggml_backend_sched_synchronize(ggml_backend_sched_t sched);
void ggml_backend_sched_set_tensor_backend(ggml_backend_sched_t sched, struct ggml_tensor *node, ggml_backend_t backend);
ggml_backend_t ggml_backend_sched_get_tensor_backend(ggml_backend_sched_t sched, struct ggml_tensor *node);
int ggml_backend_sched_get_n_backends(ggml_backend_sched_t sched);
ggml_backend_t ggml_backend_sched_get_backend(ggml_backend_sched_t sched, int i);
size_t ggml_backend_sched_get_buffer_size(ggml_backend_sched_t sched, ggml_backend_t backend);
typedef bool (*ggml_backend_sched_copy_callback)(ggml_backend_t backend, const struct ggml_tensor *src, struct ggml_tensor *dst,
                                                 struct ggml_cgraph *graph, void *user_data);
void ggml_backend_sched_set_copy_callback(ggml_backend_sched_t sched, ggml_backend_sched_copy_callback callback, void *user_data);
int64_t ggml_time_us(void);

/* ---- async transport + graph access (sysffi.rs:336-347) ---- */
void ggml_backend_synchronize(ggml_backend_t backend);
void ggml_backend_tensor_set_async(ggml_backend_t backend, struct ggml_tensor *tensor, const void *data, size_t offset, size_t size);
void ggml_backend_tensor_get_async(ggml_backend_t backend, const struct ggml_tensor *tensor, void *data, size_t offset, size_t size);

/* ---- the -ngl placement rule (backend_emit.rs:173-190): layers il >= max(n_layer_all + 1 - n_gpu_layers, 0)
 * go to the GPU, the output layer counted as layer n_layer_all; SIZE_MAX / false for n_gpu_layers <= 0 ---- */
size_t b200_gpu_layer_start(size_t n_layer_all, int32_t n_gpu_layers);
bool b200_layer_on_gpu(size_t n_layer_all, int32_t n_gpu_layers, size_t il);

#ifdef __cplusplus
}
#endif
#endif /* GGML_BASE_B200_H */
