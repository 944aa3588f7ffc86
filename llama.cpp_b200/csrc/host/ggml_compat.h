// Host-side helpers for the B200 ggml backend.
//
// The backend is compiled against the reference's public structs
// (ggml/include/ggml.h, ggml/include/ggml-backend.h, ggml/src/ggml-backend-impl.h)
// but does not link any ggml library: the few tensor-geometry helpers it needs
// are restated here from their definitions (ggml/src/ggml.c: ggml_nbytes 1166,
// ggml_row_size 1204, ggml_is_contiguous_n 1290, type_traits table 610-880).  When
// the process hosting the plugin has ggml loaded, logging is routed to its
// logger through dlsym; otherwise it goes to stderr.
#pragma once

#include "ggml.h"
#include "ggml-backend.h"
#include "ggml-backend-impl.h"

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <dlfcn.h>

#include "../kernels/kernels.h"

namespace b200 {

struct TypeGeom { int blck; int size; };
// block element count and block byte size of every ggml_type (index = enum value)
static const TypeGeom k_type_geom[GGML_TYPE_COUNT] = {
    {1, 4}, {1, 2}, {32, 18}, {32, 20}, {0, 0}, {0, 0}, {32, 22}, {32, 24}, {32, 34}, {32, 36},
    {256, 84}, {256, 110}, {256, 144}, {256, 176}, {256, 210}, {256, 292},
    {256, 66}, {256, 74}, {256, 98}, {256, 50}, {32, 18}, {256, 110}, {256, 82}, {256, 136},
    {1, 1}, {1, 2}, {1, 4}, {1, 8}, {1, 8}, {256, 56}, {1, 2},
    {0, 0}, {0, 0}, {0, 0}, {256, 54}, {256, 66}, {0, 0}, {0, 0}, {0, 0},
};

inline int64_t t_blck(int type) { return type >= 0 && type < GGML_TYPE_COUNT ? k_type_geom[type].blck : 0; }
inline size_t  t_size(int type) { return type >= 0 && type < GGML_TYPE_COUNT ? (size_t) k_type_geom[type].size : 0; }
inline bool    t_quantized(int type) { return t_blck(type) > 1; }
inline size_t  t_row_size(int type, int64_t ne) { return t_blck(type) ? t_size(type) * (size_t) (ne / t_blck(type)) : 0; }

inline int64_t t_nelements(const ggml_tensor * t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }
inline int64_t t_nrows(const ggml_tensor * t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
inline bool    t_empty(const ggml_tensor * t) { return t_nelements(t) == 0; }

inline size_t t_nbytes(const ggml_tensor * t) {
    for (int i = 0; i < GGML_MAX_DIMS; ++i) if (t->ne[i] <= 0) return 0;
    size_t nbytes;
    const int64_t blck = t_blck(t->type);
    if (blck == 1) {
        nbytes = t_size(t->type);
        for (int i = 0; i < GGML_MAX_DIMS; ++i) nbytes += (size_t) (t->ne[i] - 1) * t->nb[i];
    } else {
        nbytes = (size_t) t->ne[0] * t->nb[0] / (size_t) blck;
        for (int i = 1; i < GGML_MAX_DIMS; ++i) nbytes += (size_t) (t->ne[i] - 1) * t->nb[i];
    }
    return nbytes;
}

// contiguous for dims > n (rows may be padded up to dim n)
inline bool t_contiguous_n(const ggml_tensor * t, int n) {
    size_t next_nb = t_size(t->type);
    if (t->ne[0] != t_blck(t->type) && t->nb[0] != next_nb) return false;
    next_nb *= (size_t) (t->ne[0] / t_blck(t->type));
    for (int i = 1; i < GGML_MAX_DIMS; ++i) {
        if (t->ne[i] != 1) {
            if (i > n) {
                if (t->nb[i] != next_nb) return false;
                next_nb *= (size_t) t->ne[i];
            } else {
                next_nb = (size_t) t->ne[i] * t->nb[i];
            }
        }
    }
    return true;
}
inline bool t_contiguous(const ggml_tensor * t) { return t_contiguous_n(t, 0); }
inline bool t_same_shape(const ggml_tensor * a, const ggml_tensor * b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}
inline bool t_can_repeat(const ggml_tensor * small, const ggml_tensor * big) {
    if (t_empty(small)) return t_empty(big);
    for (int i = 0; i < GGML_MAX_DIMS; ++i) if (big->ne[i] % small->ne[i] != 0) return false;
    return true;
}

inline TensorD to_desc(const ggml_tensor * t) {
    TensorD d;
    d.data = t->data; d.type = (int) t->type;
    for (int i = 0; i < 4; ++i) { d.ne[i] = t->ne[i]; d.nb[i] = (int64_t) t->nb[i]; }
    return d;
}
inline float op_param_f32(const ggml_tensor * t, int i) { float v; memcpy(&v, (const char *) t->op_params + i * sizeof(int32_t), sizeof(v)); return v; }
inline int32_t op_param_i32(const ggml_tensor * t, int i) { return t->op_params[i]; }

// ---- logging ----
typedef void (*ggml_log_internal_t)(enum ggml_log_level, const char *, ...);
inline void log_msg(enum ggml_log_level level, const char * fmt, ...) {
    static ggml_log_internal_t host_log = (ggml_log_internal_t) dlsym(RTLD_DEFAULT, "ggml_log_internal");
    char buf[1024];
    va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof(buf), fmt, ap); va_end(ap);
    if (host_log) host_log(level, "%s", buf);
    else if (level >= GGML_LOG_LEVEL_WARN || getenv("GGML_B200_VERBOSE")) fputs(buf, stderr);
}
#define B200_LOG_INFO(...)  ::b200::log_msg(GGML_LOG_LEVEL_INFO, __VA_ARGS__)
#define B200_LOG_WARN(...)  ::b200::log_msg(GGML_LOG_LEVEL_WARN, __VA_ARGS__)
#define B200_LOG_ERROR(...) ::b200::log_msg(GGML_LOG_LEVEL_ERROR, __VA_ARGS__)

[[noreturn]] inline void fatal(const char * file, int line, const char * what, const char * detail) {
    fprintf(stderr, "ggml-b200: fatal: %s: %s (%s:%d)\n", what, detail, file, line);
    abort();
}
#define B200_CUDA_CHECK(expr)                                                             \
    do {                                                                                  \
        cudaError_t err_ = (expr);                                                        \
        if (err_ != cudaSuccess) ::b200::fatal(__FILE__, __LINE__, #expr, cudaGetErrorString(err_)); \
    } while (0)
#define B200_ASSERT(cond) do { if (!(cond)) ::b200::fatal(__FILE__, __LINE__, "assertion failed", #cond); } while (0)

}  // namespace b200
