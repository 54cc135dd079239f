// Stand-in for gdrcopy's gdrapi.h (not installed): only the types and prototypes that the original's
// gdr_mem_manager.h names.  Nothing here is ever called by the benchmark harness, which keeps its stubs and
// doorbells in cudaHostAlloc'ed mapped memory (the original's own choice for launch types other than 3 and 4).
#pragma once
#include <stddef.h>
#include <stdint.h>
struct gdr;
typedef struct gdr* gdr_t;
typedef struct gdr_mh_s { unsigned long h; } gdr_mh_t;
struct gdr_info_t { uint64_t va; uint64_t mapped_size; uint32_t page_size; uint64_t tm_cycles; uint32_t cycles_per_ms; unsigned mapped : 1; unsigned wc_mapping : 1; };
typedef struct gdr_info_t gdr_info_t;
#define GPU_PAGE_SHIFT 16
#define GPU_PAGE_SIZE (1UL << GPU_PAGE_SHIFT)
#define GPU_PAGE_OFFSET (GPU_PAGE_SIZE - 1)
#define GPU_PAGE_MASK (~GPU_PAGE_OFFSET)
extern "C" {
gdr_t gdr_open();
int gdr_close(gdr_t g);
int gdr_pin_buffer(gdr_t g, unsigned long addr, size_t size, uint64_t p2p_token, uint32_t va_space, gdr_mh_t* handle);
int gdr_unpin_buffer(gdr_t g, gdr_mh_t handle);
int gdr_get_info(gdr_t g, gdr_mh_t handle, gdr_info_t* info);
int gdr_map(gdr_t g, gdr_mh_t handle, void** va, size_t size);
int gdr_unmap(gdr_t g, gdr_mh_t handle, void* va, size_t size);
}
