/* ggml_b200_backend.h — the ggml backend plug-in face of libggml-b200.so.
 *
 * The reference's registry loads a backend with dlopen, looks up
 * ggml_backend_init / ggml_backend_score (crates/ggml/src/backend.rs:1354-1416,
 * sysffi.rs:119-122), checks api_version == 2 and then walks the vtables below.
 * Their shape is ggml-backend-impl.h's at API version 2, which the reference
 * mirrors field for field: buffer type (backend.rs:69-84), buffer (:182-203),
 * backend (:652-669), device (:960-988), registry (:1135-1142); the C mirror the
 * reference itself declares covers the registry and the first four device slots
 * (sysffi.rs:134-167), the tensor (sysffi.rs:208-227) and the op codes
 * (sysffi.rs:371-451).  A build that has the real ggml headers uses those instead
 * of this file; every vtable in the library is filled in by field name.
 */
#ifndef GGML_B200_BACKEND_H
#define GGML_B200_BACKEND_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GGML_BACKEND_API_VERSION 2
#define GGML_MAX_DIMS 4
#define GGML_MAX_OP_PARAMS 64
#define GGML_MAX_SRC 10
#define GGML_MAX_NAME 64

/* enum ggml_op values of the pinned header (sysffi.rs:371-451) used by this backend */
enum {
    GGML_OP_NONE = 0, GGML_OP_ADD = 2, GGML_OP_MUL = 7, GGML_OP_ARGMAX = 18, GGML_OP_RMS_NORM = 25, GGML_OP_MUL_MAT = 29,
    GGML_OP_MUL_MAT_ID = 30, GGML_OP_CPY = 34, GGML_OP_CONT = 35, GGML_OP_RESHAPE = 36, GGML_OP_VIEW = 37,
    GGML_OP_PERMUTE = 38, GGML_OP_TRANSPOSE = 39, GGML_OP_GET_ROWS = 40, GGML_OP_SET_ROWS = 42,
    GGML_OP_ROPE = 48, GGML_OP_FLASH_ATTN_EXT = 74, GGML_OP_UNARY = 91, GGML_OP_GLU = 100,
};

/* Ops outside ggml's enum, served only by a backend that has a tensor-parallel group attached (the decode driver
 * of llama_b200.h emits them; the reference has no multi-device graph).  TP_ALL_REDUCE: the node aliases src[0]
 * (dense F32) and holds, afterwards, the sum of src[0] over the ranks, added in rank order.  TP_ALL_GATHER:
 * src[0] is [n_local, rows], the node [n_local * ranks, rows] with rank r's slice of every row at column
 * r * n_local; src[1] is a scratch tensor of the node's size. */
enum { B200_OP_TP_ALL_REDUCE = 0x4200, B200_OP_TP_ALL_GATHER = 0x4201 };

/* enum ggml_unary_op value carried in op_params[0] of a GGML_OP_UNARY node (crates/ggml/src/ops.rs:1632-1636) */
enum { GGML_UNARY_OP_SILU = 10 };

/* enum ggml_backend_dev_type (backend.rs:1513-1523) */
enum { GGML_BACKEND_DEVICE_TYPE_CPU = 0, GGML_BACKEND_DEVICE_TYPE_GPU = 1, GGML_BACKEND_DEVICE_TYPE_IGPU = 2,
       GGML_BACKEND_DEVICE_TYPE_ACCEL = 3, GGML_BACKEND_DEVICE_TYPE_META = 4 };

/* enum ggml_backend_buffer_usage (sysffi.rs:352-357) */
enum { GGML_BACKEND_BUFFER_USAGE_ANY = 0, GGML_BACKEND_BUFFER_USAGE_WEIGHTS = 1, GGML_BACKEND_BUFFER_USAGE_COMPUTE = 2 };

typedef struct ggml_backend_buffer_type *ggml_backend_buffer_type_t;
typedef struct ggml_backend_buffer *ggml_backend_buffer_t;
typedef struct ggml_backend *ggml_backend_t;
typedef struct ggml_backend_device *ggml_backend_dev_t;
typedef struct ggml_backend_reg *ggml_backend_reg_t;
typedef struct ggml_backend_event *ggml_backend_event_t;
typedef void *ggml_backend_graph_plan_t;

/* struct ggml_tensor — sysffi.rs:208-227 (336 bytes) */
struct ggml_tensor {
    int32_t type;
    struct ggml_backend_buffer *buffer;
    int64_t ne[GGML_MAX_DIMS];
    size_t nb[GGML_MAX_DIMS];
    int32_t op;
    int32_t op_params[GGML_MAX_OP_PARAMS / sizeof(int32_t)];
    int32_t flags;
    struct ggml_tensor *src[GGML_MAX_SRC];
    struct ggml_tensor *view_src;
    size_t view_offs;
    void *data;
    char name[GGML_MAX_NAME];
    void *extra;
    char padding[8];
};

/* The leading fields of struct ggml_cgraph (ggml-impl.h); a split handed to graph_compute holds only
 * that split's nodes (crates/ggml/src/backend_sched.rs:1746-1752). */
struct ggml_cgraph {
    int size;
    int n_nodes;
    int n_leafs;
    struct ggml_tensor **nodes;
    struct ggml_tensor **grads;
    struct ggml_tensor **grad_accs;
    struct ggml_tensor **leafs;
};

/* crates/ggml/src/backend.rs:69-84 */
struct ggml_backend_buffer_type_i {
    const char *(*get_name)(ggml_backend_buffer_type_t buft);
    ggml_backend_buffer_t (*alloc_buffer)(ggml_backend_buffer_type_t buft, size_t size);
    size_t (*get_alignment)(ggml_backend_buffer_type_t buft);
    size_t (*get_max_size)(ggml_backend_buffer_type_t buft);
    size_t (*get_alloc_size)(ggml_backend_buffer_type_t buft, const struct ggml_tensor *tensor);
    bool (*is_host)(ggml_backend_buffer_type_t buft);
};
struct ggml_backend_buffer_type {
    struct ggml_backend_buffer_type_i iface;
    ggml_backend_dev_t device;
    void *context;
};

/* crates/ggml/src/backend.rs:182-203 */
struct ggml_backend_buffer_i {
    void (*free_buffer)(ggml_backend_buffer_t buffer);
    void *(*get_base)(ggml_backend_buffer_t buffer);
    int (*init_tensor)(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor);
    void (*memset_tensor)(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor, uint8_t value, size_t offset, size_t size);
    void (*set_tensor)(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor, const void *data, size_t offset, size_t size);
    void (*get_tensor)(ggml_backend_buffer_t buffer, const struct ggml_tensor *tensor, void *data, size_t offset, size_t size);
    void (*set_tensor_2d)(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor, const void *data, size_t offset, size_t size,
                          size_t n_copies, size_t stride_tensor, size_t stride_data);
    void (*get_tensor_2d)(ggml_backend_buffer_t buffer, const struct ggml_tensor *tensor, void *data, size_t offset, size_t size,
                          size_t n_copies, size_t stride_tensor, size_t stride_data);
    bool (*cpy_tensor)(ggml_backend_buffer_t buffer, const struct ggml_tensor *src, struct ggml_tensor *dst);
    void (*clear)(ggml_backend_buffer_t buffer, uint8_t value);
    void (*reset)(ggml_backend_buffer_t buffer);
};
struct ggml_backend_buffer {
    struct ggml_backend_buffer_i iface;
    ggml_backend_buffer_type_t buft;
    void *context;
    size_t size;
    int usage;
};

/* crates/ggml/src/backend.rs:652-669 (with the graph_plan slots of the C struct) */
struct ggml_backend_i {
    const char *(*get_name)(ggml_backend_t backend);
    void (*free)(ggml_backend_t backend);
    void (*set_tensor_async)(ggml_backend_t backend, struct ggml_tensor *tensor, const void *data, size_t offset, size_t size);
    void (*get_tensor_async)(ggml_backend_t backend, const struct ggml_tensor *tensor, void *data, size_t offset, size_t size);
    bool (*cpy_tensor_async)(ggml_backend_t backend_src, ggml_backend_t backend_dst, const struct ggml_tensor *src,
                             struct ggml_tensor *dst);
    void (*synchronize)(ggml_backend_t backend);
    ggml_backend_graph_plan_t (*graph_plan_create)(ggml_backend_t backend, const struct ggml_cgraph *cgraph);
    void (*graph_plan_free)(ggml_backend_t backend, ggml_backend_graph_plan_t plan);
    void (*graph_plan_update)(ggml_backend_t backend, ggml_backend_graph_plan_t plan, const struct ggml_cgraph *cgraph);
    int (*graph_plan_compute)(ggml_backend_t backend, ggml_backend_graph_plan_t plan);
    int (*graph_compute)(ggml_backend_t backend, struct ggml_cgraph *cgraph);   /* enum ggml_status */
    void (*event_record)(ggml_backend_t backend, ggml_backend_event_t event);
    void (*event_wait)(ggml_backend_t backend, ggml_backend_event_t event);
    void (*graph_optimize)(ggml_backend_t backend, struct ggml_cgraph *cgraph);
};
struct ggml_backend {
    void *guid;
    struct ggml_backend_i iface;
    ggml_backend_dev_t device;
    void *context;
};

/* crates/ggml/src/backend.rs:930-958 */
struct ggml_backend_dev_caps { bool async; bool host_buffer; bool buffer_from_host_ptr; bool events; bool mmap_support; };
struct ggml_backend_dev_props {
    const char *name;
    const char *description;
    size_t memory_free;
    size_t memory_total;
    int type;
    const char *device_id;
    struct ggml_backend_dev_caps caps;
};

/* crates/ggml/src/backend.rs:960-988, sysffi.rs:152-167 */
struct ggml_backend_device_i {
    const char *(*get_name)(ggml_backend_dev_t dev);
    const char *(*get_description)(ggml_backend_dev_t dev);
    void (*get_memory)(ggml_backend_dev_t dev, size_t *free, size_t *total);
    int (*get_type)(ggml_backend_dev_t dev);
    void (*get_props)(ggml_backend_dev_t dev, struct ggml_backend_dev_props *props);
    ggml_backend_t (*init_backend)(ggml_backend_dev_t dev, const char *params);
    ggml_backend_buffer_type_t (*get_buffer_type)(ggml_backend_dev_t dev);
    ggml_backend_buffer_type_t (*get_host_buffer_type)(ggml_backend_dev_t dev);
    ggml_backend_buffer_t (*buffer_from_host_ptr)(ggml_backend_dev_t dev, void *ptr, size_t size, size_t max_tensor_size);
    bool (*supports_op)(ggml_backend_dev_t dev, const struct ggml_tensor *op);
    bool (*supports_buft)(ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft);
    bool (*offload_op)(ggml_backend_dev_t dev, const struct ggml_tensor *op);
    ggml_backend_event_t (*event_new)(ggml_backend_dev_t dev);
    void (*event_free)(ggml_backend_dev_t dev, ggml_backend_event_t event);
    void (*event_synchronize)(ggml_backend_dev_t dev, ggml_backend_event_t event);
};
struct ggml_backend_device {
    struct ggml_backend_device_i iface;
    ggml_backend_reg_t reg;
    void *context;
};

/* crates/ggml/src/backend.rs:1135-1142, sysffi.rs:134-150 */
struct ggml_backend_reg_i {
    const char *(*get_name)(ggml_backend_reg_t reg);
    size_t (*get_device_count)(ggml_backend_reg_t reg);
    ggml_backend_dev_t (*get_device)(ggml_backend_reg_t reg, size_t index);
    void *(*get_proc_address)(ggml_backend_reg_t reg, const char *name);
};
struct ggml_backend_reg {
    int api_version;
    struct ggml_backend_reg_i iface;
    void *context;
};

/* The two symbols the registry looks up with dlsym (crates/ggml/src/backend.rs:1354-1416). */
ggml_backend_reg_t ggml_backend_init(void);
/* 0 = "not usable on this system" (no CUDA device of compute capability 10.x), else a preference score */
int ggml_backend_score(void);

/* Names served by reg->iface.get_proc_address:
 *   "b200_backend_set_cpu_threads": void (*)(ggml_backend_t, int) — the CPU thread count whose split-KV
 *   attention arithmetic FLASH_ATTN_EXT reproduces (crates/ggml/src/flash_attn.rs:841-859); default 8.
 *   "b200_backend_get_stream": void *(*)(ggml_backend_t) — the cudaStream_t the backend launches on, for
 *   callers that time graph_compute with events or order their own work after it.
 * init_backend's params string takes "cpu_threads=<n>" and "silu_wide=<0|1>" (which host's SILU to
 * reproduce, see b200_silu in ggml_b200.h; default: this host's), and three switches for launch-level
 * fusions that change no result, for side-by-side measurements: "cuda_graphs=0" (no capture / replay of
 * repeated node lists), "fuse_siblings=0" (one launch per one-row mat-mul even when several read the same
 * activations), "fuse_glue=0" (one launch per ROPE / SET_ROWS node).  The environment variables
 * B200_CUDA_GRAPHS, B200_FUSE_SIBLINGS and B200_FUSE_GLUE set to 0 do the same for every backend. */

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_BACKEND_H */
