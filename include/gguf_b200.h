/* gguf_b200.h — GGUF v3 reader and writer of libggml-b200.so.
 *
 * The reference's own: crates/ggml/src/gguf.rs:388-655 (Gguf::open over a memory map, find_key, tensor_data)
 * and crates/ggml/src/gguf_write.rs:35-193 (GgufWriter: set_kv, add_tensor, write).  Files written here are
 * byte-identical to the reference writer's for the same content, so a synthetic model saved by this library is
 * a file the reference's tools load, and the other way round.  All functions return a b200_status unless they
 * return a count; b200_last_error() has the message.
 */
#ifndef GGUF_B200_H
#define GGUF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_gguf b200_gguf;
typedef struct b200_gguf_writer b200_gguf_writer;

/* ---- reader (versions 2 and 3; one file, no splits) ---- */
int b200_gguf_open(const char *path, b200_gguf **out);
void b200_gguf_close(b200_gguf *g);
uint32_t b200_gguf_version(const b200_gguf *g);
int64_t b200_gguf_n_kv(const b200_gguf *g);
int64_t b200_gguf_n_tensors(const b200_gguf *g);
uint64_t b200_gguf_data_offset(const b200_gguf *g);
/* tensor i: name, ggml type id, ne[4], a pointer into the map, byte size (0 for a type this library does not know) */
int b200_gguf_tensor(const b200_gguf *g, int64_t i, const char **name, int *type, int64_t ne[4], const void **data, size_t *nbytes);
int b200_gguf_find_tensor(const b200_gguf *g, const char *name);   /* index or -1 */
/* keys; integer getters accept any integer width (and the first entry of a per-layer array) */
int b200_gguf_get_u32(const b200_gguf *g, const char *key, uint32_t *out);
int b200_gguf_get_f32(const b200_gguf *g, const char *key, float *out);
int b200_gguf_get_str(const b200_gguf *g, const char *key, char *out, size_t out_len);
int64_t b200_gguf_arr_len(const b200_gguf *g, const char *key);    /* -1 when missing or not an array */

/* ---- writer ---- */
int b200_gguf_writer_new(uint64_t alignment, b200_gguf_writer **out);
void b200_gguf_writer_free(b200_gguf_writer *w);
int b200_gguf_set_u32(b200_gguf_writer *w, const char *key, uint32_t v);
int b200_gguf_set_f32(b200_gguf_writer *w, const char *key, float v);
int b200_gguf_set_str(b200_gguf_writer *w, const char *key, const char *v);
/* elem_type: a GGUF scalar value type id (0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32, 7 bool, 10 u64, 11 i64, 12 f64) */
int b200_gguf_set_arr(b200_gguf_writer *w, const char *key, uint32_t elem_type, const void *data, uint64_t count);
int b200_gguf_set_arr_str(b200_gguf_writer *w, const char *key, const char *const *strs, uint64_t count);
/* data must stay valid until b200_gguf_write */
int b200_gguf_add_tensor(b200_gguf_writer *w, const char *name, int type, const int64_t ne[4], const void *data, size_t nbytes);
int b200_gguf_write(const b200_gguf_writer *w, const char *path);

#ifdef __cplusplus
}
#endif
#endif /* GGUF_B200_H */
