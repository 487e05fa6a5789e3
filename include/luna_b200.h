/*
 * C-ABI of the B200 (sm_100a) implementation of LunaEquivariance's UVU TensorProductConv hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (cudaStream_t passed as void*),
 * returns an int status (0 = success, negative = luna_status) and never throws.  Unless stated otherwise nothing
 * here allocates device memory per call: outputs and scratch are provided by the caller.  Launches are
 * asynchronous on the given stream; no call synchronises the device.
 *
 * Citations name the interface of the reference (HPC-AI-Team/LunaEquivariance v0.3.0, paths relative to its
 * root) that each entry point stands in for.
 */
#ifndef LUNA_B200_H_
#define LUNA_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define LUNA_API __attribute__((visibility("default")))
#else
#define LUNA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  LUNA_OK = 0,
  LUNA_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, inconsistent description */
  LUNA_ERR_UNSUPPORTED = -2,      /* valid request this build has no kernel for */
  LUNA_ERR_CUDA = -3,             /* a CUDA runtime call or launch failed; see luna_last_error() */
  LUNA_ERR_MISALIGNED = -4,       /* a pointer is not aligned to the element size */
  LUNA_ERR_SCRATCH = -5,          /* scratch buffer missing or too small */
  LUNA_ERR_DEVICE_TIMEOUT = -6,   /* a bounded in-kernel wait ran out (reported by luna_uvu_check_status) */
  LUNA_ERR_OVERFLOW = -7          /* sizes exceed the 32-bit graph index range */
} luna_status;

typedef enum { LUNA_F32 = 0, LUNA_F64 = 1 } luna_dtype;

/* Human-readable description of the last failure on the calling thread ("" if none). */
LUNA_API const char* luna_last_error(void);

/* Library version and the SM architecture the kernels were compiled for (100 for sm_100a). */
LUNA_API int luna_version(void);
LUNA_API int luna_compiled_sm(void);

/* --------------------------------------------------------------------------------------------------------------
 * UVU convolution plan.
 *
 * One luna_uvu_path per (instruction, edge channel v), exactly the "generated_specs" entries produced by the
 * reference's build_uvu_conv_metadata (src/lunatp/uvu_conv/kernels/utils.py:23-119):
 *   x  element (u, i) at x_offset   + u*(2*l1+1) + i        y element j at y_offset + j
 *   out element (u, k) at out_offset + u*(2*l3+1) + k        weight of channel u at weight_offset + u*weight_stride
 * and sparse coupling terms (i, j, k, c) with the path normalisation folded into c
 * (src/lunatp/utils/cg.py:31-41).  Terms of path p are term_*[term_begin .. term_end).
 */
typedef struct {
  int32_t x_offset, y_offset, out_offset, weight_offset;
  int32_t weight_stride, channels;
  int32_t l1, l2, l3;
  int32_t term_begin, term_end;
} luna_uvu_path;

typedef struct {
  int32_t dtype; /* luna_dtype of x, y, w and all outputs */
  int32_t in1_dim, in2_dim, out_dim, weight_numel;
  int32_t num_paths;
  const luna_uvu_path* paths;
  int32_t num_terms;
  const int32_t* term_i;
  const int32_t* term_j;
  const int32_t* term_k;
  const double* term_c;
} luna_uvu_desc;

typedef struct luna_uvu_plan luna_uvu_plan;

/* Stands in for LunaTPUVUConv.__init__ / configure_uvu_conv (src/lunatp/interface.py:123-144,
 * src/lunatp/uvu_conv/kernels/utils.py:121-158), which JIT-compile kernels for one configuration; here the
 * kernels are prebuilt and the plan only holds small lookup tables (host copy, plus one device copy per GPU made
 * on first use on that GPU and released by luna_uvu_plan_destroy). */
LUNA_API int luna_uvu_plan_create(const luna_uvu_desc* desc, luna_uvu_plan** plan);
LUNA_API void luna_uvu_plan_destroy(luna_uvu_plan* plan);

/* Plan queries. */
typedef enum {
  LUNA_PLAN_FAST_PATH = 0,      /* 1 if the staged (bulk-copy) kernels apply to this configuration */
  LUNA_PLAN_CHANNELS_PER_LANE = 1,
  LUNA_PLAN_CHANNEL_CHUNKS = 2,
  LUNA_PLAN_FWD_SMEM_BYTES = 3,
  LUNA_PLAN_BWD_SMEM_BYTES = 4,
  LUNA_PLAN_CANONICAL_L2 = 5,   /* highest edge-attribute degree if the path list is the full list of allowed
                                   (l1, l2, l3) couplings in standard order (kernels unrolled at compile time), else -1 */
  LUNA_PLAN_SPARSE_TERMS = 6,   /* > 0 if the plan's coupling terms have the compiled-in non-zero patterns, so the
                                   backward kernel with per-lane contraction of the edge-attribute gradient applies */
  LUNA_PLAN_BWD_VARIANT = 7     /* which first-order backward kernel aligned inputs get: a luna_bwd_variant */
} luna_plan_query;
typedef enum {
  LUNA_BWD_TABLE_DRIVEN = 0, /* one thread per output element, any configuration */
  LUNA_BWD_STAGED_TABLES = 1, /* staged kernel that reads the path list from tables */
  LUNA_BWD_ROW_STAGES = 2,    /* compiled-in coupling patterns, one warp per edge, whole weight rows staged */
  LUNA_BWD_UNIT_RING = 3      /* compiled-in coupling patterns, one warp per edge, (edge, degree) units in a ring */
} luna_bwd_variant;
LUNA_API int64_t luna_uvu_plan_query(const luna_uvu_plan* plan, int what);

/* Force the table-driven kernels (1) or let the plan choose (0, default).  For tests and comparisons. */
LUNA_API int luna_uvu_plan_set_generic(luna_uvu_plan* plan, int force_generic);

/* Graph tables of a destination-sorted edge list, as built by the reference's make_graph
 * (src/lunatp/graph.py:17-33): int32 endpoints, CSR by destination and by source, and the permutation that
 * lists edge ids grouped by source. */
typedef struct {
  int64_t num_nodes;     /* destination rows: out, g are [num_nodes, out_dim] */
  int64_t num_src_nodes; /* source rows: x, gx are [num_src_nodes, in1_dim]; 0 means "same as num_nodes".  Differs
                            when a rank holds a destination range of a partitioned graph. */
  int64_t num_edges;
  const int32_t* src;             /* [E] source row of each edge */
  const int32_t* dst;             /* [E] ascending destination row */
  const int32_t* dst_rowptr;      /* [num_nodes+1] */
  const int32_t* src_rowptr;      /* [num_src_nodes+1] */
  const int32_t* edge_ids_by_src; /* [E] */
} luna_graph;

/* Bytes of scratch the backward / double-backward entry points need for this plan and graph size (may be 0). */
LUNA_API int64_t luna_uvu_conv_scratch_bytes(const luna_uvu_plan* plan, int64_t num_nodes, int64_t num_edges);

/* out[N, out_dim] = sum over incoming edges of the weighted coupled product.  Replaces forward.run
 * (src/lunatp/uvu_conv/kernels/forward.py:1291-1343).  Every element of out is written (uncovered columns and
 * isolated nodes get zeros).  Deterministic: no atomics. */
LUNA_API int luna_uvu_conv_fwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                      void* out, void* stream);

/* First derivatives for cotangent g[N, out_dim]: gx[N, in1_dim], gy[E, in2_dim], gw[E, weight_numel]; a null
 * output is skipped.  Replaces backward.run (src/lunatp/uvu_conv/kernels/backward.py:572-681). */
LUNA_API int luna_uvu_conv_bwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y, const void* w,
                      const void* g, void* gx, void* gy, void* gw, void* scratch, int64_t scratch_bytes,
                      void* stream);

/* As luna_uvu_conv_bwd, except that gx is added to instead of written: gx[s] += dF/dx[s], and rows of sources without
 * an edge in this graph are left alone.  gy and gw are written as usual.  For callers that cut one graph's
 * destination-sorted edge list into several calls (destination sub-ranges): each call gets the slice of y, w, gy, gw
 * of its edges by pointer offset, and the calls add up the gradient of the shared source rows.  Used here to overlap
 * a halo exchange with the interior of a shard and to stream per-edge tensors from host memory chunk by chunk.  No
 * counterpart in the reference, whose backward always covers the whole graph (backward.py:572-681). */
LUNA_API int luna_uvu_conv_bwd_add_gx(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                             const void* w, const void* g, void* gx, void* gy, void* gw, void* scratch,
                             int64_t scratch_bytes, void* stream);

/* Same result as luna_uvu_conv_bwd, for callers that cannot allocate device memory and so have no scratch
 * buffer to pass: code running inside another program's step without an allocator of its own, loops that must
 * not hit cudaMalloc's device-wide synchronisation, processes whose memory pool is fixed at start-up.  No
 * counterpart in the reference (its operators allocate through torch).  The partial rows that luna_uvu_conv_bwd
 * keeps in caller scratch live in an array built into the library instead:
 *   - the array is luna_uvu_conv_noalloc_max_scratch_bytes() = 8 MiB.  It occupies that much memory on a GPU from
 *     the moment this part of the library is loaded there (with the runtime's default lazy loading: the set-up
 *     call below; with eager loading: context creation) until the process exits;
 *   - set-up, once per plan and device, with that device current, before any stream capture and outside the part
 *     of the program that must not allocate: luna_uvu_conv_noalloc_prepare(plan).  It looks up the array's device
 *     address (cudaGetSymbolAddress) and uploads the plan's lookup tables (one cudaMalloc);
 *   - luna_uvu_conv_bwd_noalloc itself performs no cudaMalloc/cudaFree and loads nothing: on a plan or device that
 *     has not been prepared it returns LUNA_ERR_INVALID_ARGUMENT instead;
 *   - a call that wants gy on a graph for which luna_uvu_conv_scratch_bytes exceeds the array is refused with
 *     LUNA_ERR_SCRATCH (without gy no scratch is used and any size is accepted);
 *   - every call on a device uses the same array, which still holds the previous call's partial rows (the kernel
 *     overwrites all rows it reads, nothing needs clearing).  Calls that overlap on one GPU race on it: issue them
 *     in stream order. */
LUNA_API int64_t luna_uvu_conv_noalloc_max_scratch_bytes(void);
LUNA_API int luna_uvu_conv_noalloc_prepare(luna_uvu_plan* plan);
LUNA_API int luna_uvu_conv_bwd_noalloc(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                              const void* w, const void* g, void* gx, void* gy, void* gw, void* stream);

/* Second derivatives.  rx, ry, rw are the cotangents of (gx, gy, gw); any may be null (= zero, never
 * materialised).  hx, hy, hw, hg receive d/d(x, y, w, g) of <rx,gx>+<ry,gy>+<rw,gw>; a null output is skipped.
 * Replaces double_backward.run (src/lunatp/uvu_conv/kernels/double_backward.py:1635-1800). */
LUNA_API int luna_uvu_conv_dbl_bwd(luna_uvu_plan* plan, const luna_graph* graph, const void* x, const void* y,
                          const void* w, const void* g, const void* rx, const void* ry, const void* rw, void* hx,
                          void* hy, void* hw, void* hg, void* scratch, int64_t scratch_bytes, void* stream);

/* Reads (and clears) the device-side status word of the plan on the current device: LUNA_OK, or
 * LUNA_ERR_DEVICE_TIMEOUT if a bounded wait inside a kernel gave up.  Synchronises the given stream. */
LUNA_API int luna_uvu_check_status(luna_uvu_plan* plan, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Graph tables.  Replaces make_graph_tables / graph_bounds (src/lunatp/utils/graph.py:637-838) for int32
 * tables.  Inputs src/dst are int32 or int64 device arrays (index_bits 32/64), dst ascending.
 * luna_graph_bounds scans the edge list and returns, after synchronising the stream, the smallest and largest
 * index of src and of dst and whether dst is unsorted (the caller raises the reference's errors from these).
 * luna_graph_build fills the tables; it trusts the bounds (indices inside [0, num_nodes) / [0, num_src_nodes)). */
typedef struct {
  int32_t* src;               /* [E] */
  int32_t* dst;               /* [E] */
  int32_t* dst_rowptr;        /* [num_nodes+1] */
  int32_t* src_rowptr;        /* [num_src_nodes+1] */
  int32_t* edge_ids_by_src;   /* [E] stable by source */
  int32_t* node_order;        /* [num_nodes] in-degree descending, stable */
  int32_t* source_node_order; /* [num_src_nodes] out-degree descending, stable */
} luna_graph_out;
LUNA_API int64_t luna_graph_scratch_bytes(int64_t num_nodes, int64_t num_edges);
LUNA_API int luna_graph_bounds(const void* src, const void* dst, int index_bits, int64_t num_edges, int64_t* min_index,
                      int64_t* max_src, int64_t* max_dst, int* unsorted, void* scratch, int64_t scratch_bytes,
                      void* stream);
LUNA_API int luna_graph_build(const void* src, const void* dst, int index_bits, int64_t num_nodes, int64_t num_src_nodes,
                     int64_t num_edges, const luna_graph_out* out, void* scratch, int64_t scratch_bytes,
                     void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Real spherical harmonics (e3nn convention), degrees <= 12.  v[n,3] -> out[n, sum(2l+1)] for the listed
 * degrees.  normalization: 0 component, 1 norm, 2 integral.  Replaces run_forward / run_backward orders 1 and 2
 * (src/o3/spherical_harmonics/kernels/forward.py:612-701, kernels/backward.py:483-553). */
typedef struct {
  int32_t dtype;
  int32_t num_degrees;
  int32_t degrees[32];
  int32_t normalize;
  int32_t normalization;
} luna_sh_desc;
LUNA_API int luna_sh_fwd(const luna_sh_desc* desc, const void* v, void* out, int64_t n, void* stream);
/* dx[n,3] = J^T g */
LUNA_API int luna_sh_bwd(const luna_sh_desc* desc, const void* v, const void* g, void* dx, int64_t n, void* stream);
/* With rx[n,3] the cotangent of dx: sx[n,3] = d<rx,dx>/dv, sg[n,C] = d<rx,dx>/dg = J rx; null outputs skipped. */
LUNA_API int luna_sh_dbl_bwd(const luna_sh_desc* desc, const void* v, const void* g, const void* rx, void* sx, void* sg,
                    int64_t n, void* stream);

/* --------------------------------------------------------------------------------------------------------------
 * Measurement aid, no counterpart in the reference: launches register-resident chains of fused multiply-adds
 * (kind 0: packed FP32 pairs, the instruction the FP32 kernels run on; kind 1: FP64) and returns the FLOPs the
 * launch performs in *flops.  Timed by the caller with events on `stream`, it gives the GPU's measured arithmetic
 * peak, the denominator of the arithmetic roofline.  sink: device buffer of at least 1025 doubles. */
LUNA_API int luna_probe_fma(int kind, int iterations, void* sink, double* flops, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUNA_B200_H_ */
