/* b200_nvfp4.h -- C ABI of the B200 (sm_100a) NVFP4 weight-path library, libb200nvfp4.so.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its comment says
 * host; every call enqueues on `stream` and returns without synchronising unless its comment says
 * otherwise.  Return value: 0 on success, a B200_E* code otherwise (b200_nvfp4_strerror names it).
 * There is no CPU fallback.  Buffers belong to the caller; what the library itself holds is:
 *   - cached device attributes and encoded TMA tensor maps of the weights it has seen (host memory)
 *   - per GPU: the status word of the bounded waits, the job counters of the byte accounting, and
 *     the 1 MiB static scratch of b200_moe_forward_static
 *   - per prepared MoE layer: its tensor maps in device memory (b200_moe_prepare .. b200_moe_release)
 *   - per expert-parallel context: its buffers, streams, events and NCCL communicator
 *   - the process-wide options (b200_nvfp4_set_option) and the byte-credit callback
 *
 * NVFP4 tensor = three buffers (reference include/nvfp4.cuh:3-7):
 *   packed [N, K/2] u8, low nibble = even k;  scale [N, K/16] u8 fp8-e4m3;  gscale [1] f32
 *   w[n,k] = e2m1(nibble) * e4m3(scale[n,k/16]) / gscale[0]
 * Activations and outputs are fp32 row-major: x[M,K], y[M,N].
 */
#ifndef B200_NVFP4_H
#define B200_NVFP4_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200_stream;      /* same type as cudaStream_t */

enum {
    B200_OK = 0,
    B200_EINVAL = 1,      /* null pointer, non-positive size, M out of range */
    B200_ESHAPE = 2,      /* K not a multiple of 16, or a shape the kernel cannot tile */
    B200_EALIGN = 3,      /* pointer below the 4-byte floor the format guarantees */
    B200_ELAUNCH = 4,     /* the CUDA runtime refused the launch (cudaGetLastError text logged) */
    B200_ELIMIT = 5,      /* size beyond a documented maximum */
    B200_ENOTIMPL = 6,
    B200_ETIMEOUT = 7,    /* a bounded host-side wait ran out (expert-parallel exchange) */
    B200_ECOMM = 8        /* NCCL is missing or returned an error */
};
enum { B200_F32 = 0, B200_BF16 = 1 };          /* dtype of a non-quantised weight (gemv.h:13) */
enum { B200_GEMV_MULTI_MAX = 8, B200_GEMV_M_MAX = 8 };

/* Weight handle.  Mirrors glm5::WRef (reference include/gemv.h:16-26): a plain row-major
 * [N,K] buffer of `dtype`, or an NVFP4 triple, which wins whenever `packed` is non-null. */
typedef struct {
    const void*    p;
    const uint8_t* packed;
    const uint8_t* scale;
    const float*   gscale;
} b200_wref;

/* One gemv of a fused group.  Mirrors glm5::GemvJob (reference include/gemv.h:50-55);
 * x is [M,K], y is [M,N] for the M given to the call. */
typedef struct {
    float*       y;
    b200_wref    W;
    const float* x;
    int          N;
} b200_gemv_job;

/* Mirrors glm5::Nvfp4Mat (reference include/moe.h:13-17). */
typedef struct {
    const uint8_t* packed;
    const uint8_t* scale;
    const float*   gscale;
} b200_nvfp4_mat;

/* Alignment of an expert's tensors: packed bytes and gscale 4-byte aligned (the floor the reference's
 * checkpoint guarantees, kernels/moe.cu:167-174, 628-636), scales at any address.  The CUDA-core expert
 * kernels take 16-byte loads where a tensor allows it and 4-byte loads where not; b200_moe_prepare (the
 * tensor-core experts) wants every tensor 16-byte aligned and answers B200_ENOTIMPL otherwise.
 * Mirrors glm5::MoeLayer (reference include/moe.h:19-26) plus the geometry the reference
 * bakes in at compile time (include/glm5_config.h:20, 84-91), here per layer at run time. */
typedef struct {
    b200_wref             router_w;      /* bf16 [n_expert, hidden] */
    const float*          router_bias;   /* f32 [n_expert] */
    const b200_nvfp4_mat* experts;       /* DEVICE array, 3*n_expert: [3e]=gate [3e+1]=up [3e+2]=down */
    const b200_nvfp4_mat* shared;        /* DEVICE array of 3, or null for no shared expert */
    int   n_expert;
    int   topk;                          /* <= 16 */
    int   hidden;                        /* multiple of 32 */
    int   inter;                         /* multiple of 32 */
    float routed_scale;                  /* 2.5 in the reference */
    float swiglu_limit;                  /* 10 in the reference */
    int   norm_topk;                     /* 1: renormalise the selected gates */
} b200_moe_layer;

const char* b200_nvfp4_strerror(int code);
int         b200_nvfp4_version(void);

/* Every wait inside a kernel of this library is bounded.  If one ever runs out, the kernel
 * records (site << 16 | block) in a per-device status word and carries on to termination; the
 * outputs of that launch are then undefined.  This call SYNCHRONISES the device copy of that
 * word into *out (host pointer; 0 = nothing happened) and optionally clears it.  No counterpart
 * in the reference, whose kernels never wait on one another. */
int b200_nvfp4_device_status(unsigned int* out, int clear);

/* Self-test of that mechanism: enqueues one small kernel whose only thread waits on a barrier nobody
 * arrives at.  The wait runs out after its limit (about a second), the kernel returns normally, and
 * b200_nvfp4_device_status then reports site 15 (0x000f0000 | block 0).  The context stays usable. */
int b200_nvfp4_selftest_bounded_wait(b200_stream stream);

/* Process-wide options.  B200_OPT_STABLE_WEIGHTS = 1 declares that no kernel running on a
 * stream writes NVFP4 weight buffers that a later call on that stream reads (true for an
 * inference engine, whose weights are loaded once).  The pipelined kernels, which are launched
 * with programmatic stream serialisation, may then start copying weights while the previous
 * kernel of the stream is still finishing; activations, scales and outputs are still only
 * touched after the previous kernel has completed.  Default 0 (also settable with the
 * environment variable B200_STABLE_WEIGHTS=1).  No counterpart in the reference. */
/* B200_OPT_PREFILL_FP4 (default 1; environment B200_PREFILL_FP4=0 turns it off): calls that carry
 * scratch and 16 or more activation rows -- b200_nvfp4_gemm_ws with M >= 16, the MoE block with 16
 * or more tokens on a prepared layer -- run the wide tensor-core GEMM, which quantises the
 * activations to NVFP4 per token (see b200_nvfp4_gemm_bf16 for what that costs in accuracy).  With
 * 0 those calls keep fp32-activation accuracy at every M: b200_nvfp4_gemm_ws through the exact wide GEMM
 * (b200_nvfp4_gemm_bf16_exact), the MoE block in passes of 8 rows over the experts. */
enum { B200_OPT_STABLE_WEIGHTS = 1, B200_OPT_PREFILL_FP4 = 2 };
int b200_nvfp4_set_option(int option, int value);

/* Byte accounting for a host-side profiler.  The reference's launch sites credit the weight bytes they
 * read to its profiler (dprof_bytes: kernels/gemv.cu:377, 427, 458, 677; kernels/moe.cu:656-667, 719-722;
 * include/dprof.h:83-103), because a weight read at width M serves M tokens and the MoE count depends on
 * the routing.  This library reports the same quantity through a callback: `fn(kind, bytes, user)` is
 * called on the calling host thread at every launch site with the weight bytes THAT call reads -- for an
 * NVFP4 product passes * N * K * 0.5625 (passes = how often this library streams W for the call's M),
 * for the MoE experts up to 8 tokens pairs * 3 * inter * hidden * 0.5625 split into its gate/up and
 * down halves.  Where rows are grouped by expert on the device (more than 8 tokens) the count is only
 * known there: it accumulates in a device counter that b200_nvfp4_flush_byte_credit reads (this
 * SYNCHRONISES), credits (credit != 0) or discards (credit == 0, after a warm-up), and clears -- the
 * contract of the reference's dprof_set_flush.  A drop-in build's callback simply forwards to dprof_bytes /
 * dprof_bytes_to.  NULL switches the reporting off (the default). */
enum { B200_CREDIT_GEMM = 0, B200_CREDIT_MOE_ROUTER = 1, B200_CREDIT_MOE_ACT = 2, B200_CREDIT_MOE_DOWN = 3 };
typedef void (*b200_byte_credit_fn)(int kind, double bytes, void* user);
int b200_nvfp4_set_byte_credit(b200_byte_credit_fn fn, void* user);
int b200_nvfp4_flush_byte_credit(int credit);

/* y[M,N] = x[M,K] . W[N,K]^T.  Replaces glm5::gemm / glm5::gemv (reference include/gemv.h:29,
 * 75; kernels/gemv.cu:369-396, 456-465, 649-701).  Any M >= 1: rows are processed in chunks of
 * up to 8 and W is re-read once per chunk.  Each output row of y depends only on its own row
 * of x, and the result is bit-identical from run to run. */
int b200_nvfp4_gemm(float* y, const b200_wref* W, const float* x, int M, int N, int K,
                    int dtype, b200_stream stream);

/* n (1..8) gemvs that share K, M (1..8) and dtype, in ONE launch; jobs is a HOST array.
 * Replaces glm5::gemv_multi (reference include/gemv.h:56, kernels/gemv.cu:404-435), widened
 * from 4 jobs at M=1 to 8 jobs at M<=8.  Bit-identical to n separate b200_nvfp4_gemm calls. */
int b200_nvfp4_gemv_multi(const b200_gemv_job* jobs, int n, int M, int K, int dtype,
                          b200_stream stream);

/* The two calls above with scratch from the caller, for M >= 2: the activation rows are split into
 * their tensor-core operand image once, by one small launch into `ws`, instead of by every CTA of
 * the product kernel (which is what makes rows beyond the first cost 2.4 us each otherwise).
 * ws: b200_nvfp4_split_workspace_bytes(M, K) bytes of device memory, 256-byte aligned; only this
 * call's kernels use it, so calls that may overlap on the GPU need separate scratch, and the
 * next call on the same stream may reuse it.  Results are bit-identical to the plain calls.
 * gemv_multi_ws wants all jobs to share one x; where the scratch cannot be used (M = 1, shapes the
 * tensor-core kernel does not take, ws == NULL) these run exactly as the plain calls.  No
 * counterpart in the reference, whose gemm has no workspace argument (include/gemv.h:75).
 * With M >= 16 and B200_OPT_PREFILL_FP4 on (the default), b200_nvfp4_gemm_ws runs the wide GEMM of
 * b200_nvfp4_gemm_bf16 on the f32 rows instead (W read once per 256 rows, activations quantised to
 * NVFP4 per token): the scratch size below covers it. */
size_t b200_nvfp4_split_workspace_bytes(int M, int K);
int b200_nvfp4_gemm_ws(float* y, const b200_wref* W, const float* x, int M, int N, int K,
                       int dtype, void* ws, b200_stream stream);
int b200_nvfp4_gemv_multi_ws(const b200_gemv_job* jobs, int n, int M, int K, int dtype,
                             void* ws, b200_stream stream);

/* The wide GEMM, for prefill and batched widths (M >= 16; any M >= 1 is accepted):
 * y[M,N] (f32) = x[M,K] (bf16) . W[N,K]^T on tcgen05.mma kind::mxf4nvf4 with BOTH operands in NVFP4.
 * W is read once for up to 256 rows of x (the reference's gemm streams W once per chunk of 4 rows,
 * kernels/gemv.cu:369-396, include/gemv.h:65-75).  The activations are quantised to NVFP4 first, one
 * token at a time (b200_nvfp4_quantize_tokens below), which costs about 9 % per-element activation
 * error: results match deq(W) . deq(quant(x)) to 1e-3 and deviate from the exact product by a few
 * per cent.  Callers that need fp32-activation accuracy use b200_nvfp4_gemm.  A token's result does
 * not depend on the other rows of the batch.  Needs K % 256 == 0, K <= 16384, 16-byte aligned W and x;
 * otherwise B200_ENOTIMPL.  ws: b200_nvfp4_gemm_bf16_workspace_bytes(M, K) bytes, 256-byte aligned,
 * used only by this call's kernels.  No counterpart in the reference, which has no bf16-activation
 * or tensor-core entry point. */
size_t b200_nvfp4_gemm_bf16_workspace_bytes(int M, int K);
int b200_nvfp4_gemm_bf16(float* y, const b200_wref* W, const void* x_bf16, int M, int N, int K,
                         void* ws, b200_stream stream);

/* The EXACT wide GEMM: the same call with fp32-activation accuracy.  The NVFP4 weights are dequantised to
 * fp16 inside the kernel (e2m1 * e4m3 is an fp16 number), the bf16 activations are scaled per token by a
 * power of two into fp16, and the products run on tcgen05.mma kind::f16 with fp32 accumulation: results
 * match the reference's fp32-activation gemm (kernels/gemv.cu:246-329) to fp32 rounding (measured
 * rel-L2 < 1e-6), W still crosses HBM once per call, and the tensor pipe runs at the bf16 rate instead
 * of the FP4 rate.  Same shape and alignment conditions as b200_nvfp4_gemm_bf16; ws:
 * b200_nvfp4_gemm_bf16_exact_workspace_bytes(M, K) bytes.  b200_nvfp4_gemm_ws takes this path for
 * M >= 16 when B200_OPT_PREFILL_FP4 is 0 (f32 rows are then rounded to fp16 once: rel-L2 about 1.4e-4).
 * No counterpart in the reference. */
size_t b200_nvfp4_gemm_bf16_exact_workspace_bytes(int M, int K);
int b200_nvfp4_gemm_bf16_exact(float* y, const b200_wref* W, const void* x_bf16, int M, int N, int K,
                               void* ws, b200_stream stream);

/* Per-token activation quantiser of the wide GEMM: every row of x[M,K] (bf16 when x_is_f32 == 0, else
 * f32) is quantised with the reference's quant_block rule (tools/requant_dense_nvfp4.py:53-68) and its
 * own global scale gs[m] = 2688 / max(amax(row m), 1e-12) (:215 per row); bit-exact with that rule.
 * packed [M, K/2]; scale is STEP-MAJOR, [K/256][M][16] (the 16 scale bytes of one row for 256
 * consecutive k are contiguous); gs f32 [M].  K % 256 == 0. */
int b200_nvfp4_quantize_tokens(const void* x, int x_is_f32, int M, int K, uint8_t* packed,
                               uint8_t* scale_step_major, float* gs, b200_stream stream);

/* The dense-layer MLP in one call: y[M,hidden] = down . ( silu(min(gate.x, limit)) * clamp(up.x, -limit, limit) ).
 * Replaces glm5::dense_mlp / dense_mlp_batch (reference kernels/layer.cu:235-254, k_swiglu_clamped :201-208).
 * gate, up: NVFP4 [inter, hidden]; down: NVFP4 [hidden, inter].  gate and up run as one fused two-job launch up
 * to 8 rows; from 16 rows on the products follow b200_nvfp4_gemm_ws (wide GEMM unless B200_OPT_PREFILL_FP4 is 0).
 * ws: b200_dense_mlp_workspace_bytes(M, hidden, inter) bytes, 256-byte aligned (the reference's caller passes
 * 2 * M * inter floats; this needs the split scratch as well). */
size_t b200_dense_mlp_workspace_bytes(int M, int hidden, int inter);
int b200_dense_mlp(const float* x, const b200_wref* gate, const b200_wref* up, const b200_wref* down,
                   int hidden, int inter, float limit, float* y, void* ws, int M, b200_stream stream);

/* Element-wise converters (reference include/gemv.h:61-62, kernels/gemv.cu:470-488). */
int b200_f32_to_bf16(void* dst_bf16, const float* src, size_t n, b200_stream stream);
int b200_bf16_to_f32(float* dst, const void* src_bf16, size_t n, b200_stream stream);

/* bf16 [N,K] -> NVFP4 triple, bit-exact with the reference quantiser (tools/
 * requant_dense_nvfp4.py:53-68 quant_block and :209-215 global scale).  Outputs are caller
 * allocated: packed N*K/2 bytes, scale N*K/16 bytes, gscale 4 bytes.  If `gscale_in` is
 * non-null the tensor pass is skipped and that scale is used (activation re-quantisation). */
int b200_nvfp4_quantize(const void* w_bf16, int N, int K, uint8_t* packed, uint8_t* scale,
                        float* gscale, const float* gscale_in, b200_stream stream);

/* NVFP4 triple -> fp32 [N,K] (reference ref/gen_moe.py:23-30); a test and tooling helper. */
int b200_nvfp4_dequantize(float* out, const b200_nvfp4_mat* W, int N, int K, b200_stream stream);

/* Workspace for M tokens of one MoE layer, in bytes (reference include/moe.h:28-29,
 * kernels/moe.cu:602, 621-625 count floats; the drop-in header converts). */
size_t b200_moe_workspace_bytes(const b200_moe_layer* L, int M);

/* Router only: logits[M,E] = x.Wr^T, sel int32 [M,topk] in descending (score+bias) order,
 * wts f32 [M,topk] (reference include/moe.h:34-35, 44-45; kernels/moe.cu:126-156, 638-650). */
int b200_moe_route(const float* x, const b200_moe_layer* L, int32_t* sel, float* wts,
                   float* logits, int M, b200_stream stream);

/* Whole block, M tokens: route, top-k SwiGLU experts, shared expert, gate-weighted sum in a
 * fixed order (reference include/moe.h:32-33, 41-43; kernels/moe.cu:669-740).  x,y [M,hidden];
 * sel/wts [M,topk] are outputs; ws holds b200_moe_workspace_bytes(L, M) bytes. */
int b200_moe_forward(const float* x, const b200_moe_layer* L, float* y, int32_t* sel,
                     float* wts, void* ws, int M, b200_stream stream);

/* Optional, once per layer after its weights are on the device: lets b200_moe_forward and
 * b200_moe_experts run their experts on the tensor-core kernels (every pair on its own up to 8
 * tokens, rows grouped by expert beyond).  It reads the layer's
 * device-side expert tables (a synchronous copy: call it at load time, never under stream
 * capture), encodes TMA descriptors for every expert and keeps them in device memory until
 * b200_moe_release or process exit.  The layer is recognised later by its experts / shared
 * pointers and geometry, so the tables and the weights must stay where they are.  Returns
 * B200_ENOTIMPL when the geometry or alignment does not suit those kernels (hidden and inter
 * multiples of 256, 16-byte aligned tensors); the layer then keeps using the CUDA-core kernels,
 * as does every layer that was never prepared.  No counterpart in the reference, whose engine
 * builds its tables at load (src/engine.cu:168-195) -- the natural place to call this. */
int b200_moe_prepare(const b200_moe_layer* L);
int b200_moe_release(const b200_moe_layer* L);

/* Expert half only, routing supplied by the caller (sel/wts are inputs).  No counterpart in
 * the reference, which always routes itself; used where routing is decided elsewhere. */
int b200_moe_experts(const float* x, const b200_moe_layer* L, float* y, const int32_t* sel,
                     const float* wts, void* ws, int M, b200_stream stream);

/* b200_moe_forward without a workspace argument, for hosts that cannot allocate one: an engine
 * whose buffers were sized at start-up by the reference's own moe_workspace_floats(), and which
 * may not call cudaMalloc later (it would synchronise the device in the middle of the token
 * loop, and is illegal under stream capture).  The scratch is a 1 MiB array inside the library
 * (b200_moe_static_ws_limit()), held by every GPU that loads the library until exit; it holds the
 * router logits [M, n_expert] and the activations [M, topk + 1, inter] (f32, each part rounded up
 * to 256 bytes: 14 tokens at the reference geometry), and a layer / M that needs more is refused with B200_ELIMIT.  This entry point
 * always runs the CUDA-core expert kernels, prepared layer or not.  The call allocates
 * nothing.  The FIRST call on each device looks the array's device address up
 * (cudaGetSymbolAddress) -- make that call before any stream capture.  All calls on a device
 * share the array and it keeps the last call's contents; nothing in it needs clearing, but two
 * calls that overlap on the GPU race on it, so keep them on one stream or order them.
 * This entry point has no counterpart in the reference. */
size_t b200_moe_static_ws_limit(void);
int b200_moe_forward_static(const float* x, const b200_moe_layer* L, float* y, int32_t* sel,
                            float* wts, int M, b200_stream stream);

/* ---- safetensors overlay of NVFP4 triples (host side; no GPU involved) ---------------------------
 * The wire format of the reference's requant tool (tools/requant_dense_nvfp4.py:123-152 ShardWriter,
 * :224-239): per selected tensor `<stem>.weight` the three tensors `<stem>.weight_packed` (U8),
 * `.weight_scale` (F8_E4M3), `.weight_global_scale` (F32) in shards overlay-%05d.safetensors whose data
 * and every tensor start on 16-byte boundaries, plus model.safetensors.index.json.  The writer emits the
 * same bytes as that tool for the same tensors in the same order, so an overlay requantised on the GPU
 * (b200_nvfp4_quantize, copied back) loads through the reference's own loader (include/safetensors.h:54-113,
 * include/weight_store.h:23-33).  packed / scale are HOST buffers; a new shard starts once the current
 * one holds shard_bytes (0 = the tool's default, 2 GiB).  close writes the last shard and the index.
 * b200_overlay_family: index of the first family of `families_csv` (NULL = the arch's default list) whose
 * pattern matches the tensor name (:76-120, arch "glm5" or "mimo"), -1 = not selected, -2 = unknown name.
 * The reader maps an overlay directory and hands out host pointers to a triple (valid until close). */
typedef struct b200_overlay_writer b200_overlay_writer;
typedef struct b200_overlay b200_overlay;
typedef struct { const uint8_t* packed; const uint8_t* scale; float gscale; int N; int K; } b200_overlay_entry;
int b200_overlay_writer_open(b200_overlay_writer** out, const char* dir, uint64_t shard_bytes);
int b200_overlay_writer_add(b200_overlay_writer* w, const char* tensor_name, const uint8_t* packed,
                            const uint8_t* scale, float gscale, int N, int K);
int b200_overlay_writer_close(b200_overlay_writer* w);
int b200_overlay_family(const char* arch, const char* families_csv, const char* tensor_name);
int b200_overlay_open(b200_overlay** out, const char* dir);
int b200_overlay_count(const b200_overlay* o);
int b200_overlay_find(const b200_overlay* o, const char* tensor_name, b200_overlay_entry* out);
int b200_overlay_close(b200_overlay* o);

/* ---- expert-parallel MoE layer (one process per GPU, NCCL) ------------------------------------
 * The reference has no multi-GPU form (all experts sit behind one device table, src/engine.cu:168-195);
 * this is the same block (kernels/moe.cu:669-740, fixed-order gate sum :584-597) with the experts of a
 * layer sharded over `world` GPUs of one node: rank r owns experts [r*E/world, (r+1)*E/world), router,
 * bias and shared expert are replicated, tokens are data-parallel.  Per call: route, one NCCL
 * all-gather of the per-destination counts, ONE grouped ncclSend/ncclRecv round that carries token rows
 * (bf16) and expert ids in the same message, the local experts on the received rows, one reverse round
 * with the f32 output rows, and the gate-weighted sum in slot order plus the shared expert (which runs on
 * a second stream and overlaps the exchange).  Token rows travel as bf16: a token's expert inputs are
 * its values rounded to bf16.
 *
 * b200_ep_unique_id: rank 0 fills 128 bytes (HOST) that the caller hands to every rank by its own means.
 * b200_ep_create: allocates the context's device buffers for up to max_tokens local tokens per call
 *   (worst case: every pair of every rank lands on this rank) and joins the NCCL communicator (a
 *   collective call: every rank must make it).  `router`: the layer's router and bias over ALL E experts
 *   (its expert tables are never read); `local`: this rank's E/world experts as a layer with topk = 1
 *   (call b200_moe_prepare on it first to get the tensor-core experts); `shared`: one expert, topk = 1,
 *   or NULL.  The tables and weights must outlive the context.  world == 1 needs no NCCL and no id.
 * b200_ep_forward: x, y [T, hidden] f32, sel/wts [T, topk] outputs, all on this rank.  With world > 1 the
 *   call waits on the host (bounded, 20 s) for the exchange sizes, so it cannot be captured in a CUDA
 *   graph; B200_ETIMEOUT means a peer never joined, and the communicator has been aborted.
 * libnccl.so.2 is bound at run time, on the first context with world > 1. */
typedef struct b200_ep b200_ep;
typedef struct {
    int tokens, recv_rows, sent_remote_rows, recv_remote_rows, local_experts_touched, pad;
    unsigned long long dispatch_bytes_out, combine_bytes_in;      /* bytes that crossed NVLink for this rank's tokens */
    float plan_us, dispatch_us, experts_us, combine_us, total_us; /* device time of the last call's phases (CUDA events) */
    float pad2;
} b200_ep_stats;
int b200_ep_unique_id(void* id128);
int b200_ep_create(b200_ep** out, const void* id128, int rank, int world, const b200_moe_layer* router,
                   const b200_moe_layer* local, const b200_moe_layer* shared, int max_tokens);
int b200_ep_forward(b200_ep* ep, const float* x, float* y, int32_t* sel, float* wts, int T,
                    b200_stream stream);
int b200_ep_last_stats(const b200_ep* ep, b200_ep_stats* out);     /* synchronises the device */
int b200_ep_destroy(b200_ep* ep);

#ifdef __cplusplus
}
#endif
#endif /* B200_NVFP4_H */
