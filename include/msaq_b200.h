/*
 * msaq_b200.h -- C ABI of the B200 (sm_100a) MSAQ-signed decode path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches on that stream, allocates
 * nothing, never synchronises the host, and returns MSAQ_OK or a negative
 * error code; msaq_last_error() gives the message of the calling thread's last
 * failure.  Scratch memory is a caller-owned workspace whose size the matching
 * *_workspace() query returns.
 *
 * Packed data layout (unchanged from the reference, ms_lib/pack.py:101-137 and
 * :479-504).  BLOCK = 32, nb = K/32 (or D/32), wbits = 8-u,
 * UB = 32*wbits/8, SB = ceil((32/gs)*u/8):
 *   weights   scale_exp int8 [nb,OUT]
 *             row-major    upper u8 [nb,UB,OUT]   shared u8 [nb,SB,OUT]
 *             column-major upper u8 [nb,OUT,UB]   shared u8 [nb,OUT,SB]
 *   KV cache  scale_exp int8 [B*Hkv,nb,Lcap]
 *             upper u8 [B*Hkv,nb,Lcap,UB]   shared u8 [B*Hkv,nb,Lcap,SB]
 * Inside a block, upper code k sits at bits [k*wbits,(k+1)*wbits) and the shared
 * code of group g = k/gs at bits [g*u,(g+1)*u) of the little-endian byte run,
 * both two's complement; value = (up*2^u + sh) * 2^scale_exp.
 *
 * Supported: u in {2,3,4}; gs in {2,4,8,16,32}; D a power of two in [32,256].
 */
#ifndef MSAQ_B200_H
#define MSAQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSAQ_OK               0
#define MSAQ_ERR_ARG         -1   /* null pointer, bad size, misaligned pointer   */
#define MSAQ_ERR_UNSUPPORTED -2   /* (u, gs, D) outside the supported set         */
#define MSAQ_ERR_WORKSPACE   -3   /* workspace missing or too small               */
#define MSAQ_ERR_CUDA        -4   /* a CUDA runtime call or a launch failed       */
#define MSAQ_ERR_DEVICE      -5   /* the current device is not an sm_100 part     */

/* Library version (major*1000 + minor). */
int msaq_version(void);
/* Message of the calling thread's most recent error ("" if none). */
const char* msaq_last_error(void);
/* Number of kernels this library has launched in the calling process. */
unsigned long long msaq_launch_count(void);

/* Process-wide options (no reference counterpart; the reference reads MS_* environment flags per call,
 * csrc/kv_attention.cu:2082-2083).  msaq_set_option returns MSAQ_OK or MSAQ_ERR_ARG; msaq_get_option the value.
 *
 * MSAQ_OPT_CHAINED_LAUNCH (default 1; MSAQ_CHAINED_LAUNCH=0 in the environment turns it off): kernels are
 *   launched with programmatic stream serialisation, so the launch and prologue of one kernel overlap the
 *   tail of the kernel before it.  Results do not change: every kernel waits for its predecessor before it
 *   reads or writes anything another kernel produces or consumes.
 * MSAQ_OPT_TENSOR_MEMORY (default 1): batched GEMVs (u=4, gs=2, 9 rows and more) run on the tcgen05 tensor
 *   cores with accumulators in tensor memory; 0 keeps them on the warp-level integer MMA path (the two paths
 *   agree to the output tolerance, not bit for bit).
 * MSAQ_OPT_INKERNEL_STAGING (default 1): small integer-MMA GEMVs (up to four rows, no fused prologue, at most
 *   eighteen K blocks per thread block) convert their activations inside the main kernel, one launch per GEMV; 0
 *   runs the separate staging kernel in front, as all other launches do.  Same staged values either way.
 * MSAQ_OPT_WAIT_POLLS (default 2^20): poll limit of every wait on a shared-memory barrier inside the pipelined
 *   kernels.  A wait that reaches it gives up: the kernel finishes by itself, the outputs the wait fed become
 *   NaN, and a bit is set in the status word msaq_wait_status() reads.
 * MSAQ_OPT_TEST_SKIP_STAGE (default -1 = off; a test hook, not for production): the copy-issuing thread of
 *   the first thread block of the pipelined GEMV / flash-decode kernels stops before this pipeline stage, so
 *   that the wait for it runs out.  Used to check the give-up path without faulting or hanging anything.
 * MSAQ_OPT_EARLY_WEIGHTS (default 0): the integer-MMA GEMVs start fetching their packed weights BEFORE they wait
 *   for the kernel in front of them in the stream (only the activations wait), and every kernel of the library
 *   asks for the largest shared-memory split so that a GEMV's thread blocks can take their places on an SM while a
 *   small kernel in front still runs there.  The contract that makes this safe is the caller's: set it only
 *   where the weight planes are complete before the GEMV is enqueued -- packed at load time and synchronised
 *   since, the serving case -- never where a kernel still in flight on the stream writes them.  Three quarters
 *   through its copies a GEMV thread block then lets the kernels behind it be scheduled, so that the next GEMV's
 *   blocks take the places of blocks that have finished and fetch their first weights during this GEMV's tail.
 *   Measured on the 70B layer step: 178.8 -> 172.3 us on one GPU, 84.5 -> 80.6 us on an 8-GPU shard.  Results do
 *   not change. */
#define MSAQ_OPT_CHAINED_LAUNCH 1
#define MSAQ_OPT_TENSOR_MEMORY 2
#define MSAQ_OPT_WAIT_POLLS 3
#define MSAQ_OPT_TEST_SKIP_STAGE 4
#define MSAQ_OPT_INKERNEL_STAGING 5
#define MSAQ_OPT_EARLY_WEIGHTS 6
int msaq_set_option(int option, int value);
int msaq_get_option(int option);

/* Status word of the current device (no reference counterpart; the reference's kernels have no waits that can
 * give up).  Bits: 1 = a wait gave up in the integer-MMA GEMV, 2 = in the tensor-memory GEMV, 4 = in the
 * flash-decode kernel, 8 = an append position read from device memory was outside [0, Lcap) and the row was
 * skipped.  The call synchronises `stream`, stores the word in *status_out and, when clear != 0, resets it.
 * Do not call it while `stream` is being captured. */
#define MSAQ_STATUS_WAIT_GEMV 1
#define MSAQ_STATUS_WAIT_GEMV_TM 2
#define MSAQ_STATUS_WAIT_KV_DECODE 4
#define MSAQ_STATUS_BAD_APPEND_POS 8
#define MSAQ_STATUS_PEER_TIMEOUT 16     /* a rank's peers did not arrive in msaq_peer_exchange */
int msaq_wait_status(int clear, void* stream, int* status_out);

/* ------------------------------------------------------------------ GEMV -- */

/* Bytes of workspace the three GEMV entry points need for these sizes. */
size_t msaq_wonly_gemv_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs);

/*
 * y[OUT] = x[K] . dequant(W)^T on ROW-MAJOR planes.  x, y bf16; fp32 accumulate.
 * Replaces op `msaq::wonly_gemv` (csrc/pybind.cpp:199-200, host
 * csrc/w_gemv.cu:1410-1454).  y_f32 (optional, may be NULL) also receives the
 * result before the bf16 rounding.
 */
int msaq_wonly_gemv(const void* x, const int8_t* scale_exp, const uint8_t* upper,
                    const uint8_t* shared, void* y, float* y_f32,
                    int64_t OUT, int64_t NB, int u, int gs,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Same product on COLUMN-MAJOR planes (upper_cm / shared_cm).
 * Replaces op `msaq::wonly_gemv_wide` (csrc/pybind.cpp:201-202, host
 * csrc/w_gemv.cu:1457-1510).
 */
int msaq_wonly_gemv_wide(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm,
                         const uint8_t* shared_cm, void* y, float* y_f32,
                         int64_t OUT, int64_t NB, int u, int gs,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * Y[M,OUT] = X[M,K] . dequant(W)^T on column-major planes, any M >= 1.
 * (The tensor-memory kernel -- 9 rows and more, and the u = 2, 3 formats at gs = 2 -- widens q * 2^e through an
 * fp32 constant of about 2^23 * 2^e: block exponents above 104 overflow there.  bf16 weights of magnitude below
 * 2^110 never produce them.)
 * Replaces op `msaq::wonly_gemv_batched` (csrc/pybind.cpp:205-206, host
 * csrc/w_gemv.cu:1514-1570).
 */
int msaq_wonly_gemv_batched(const void* X, const int8_t* scale_exp, const uint8_t* upper_cm,
                            const uint8_t* shared_cm, void* Y, float* Y_f32,
                            int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * GEMV with the decoder-layer glue that precedes it folded into the activation staging (no reference
 * counterpart: the reference runs these steps as separate torch ops, tests/harness_batchsweep.py:230-243).
 *   MSAQ_PRO_NONE         y = W x                                      x [M][K]
 *   MSAQ_PRO_RMSNORM      y = W bf16(rmsnorm(x, eps))                  x [M][K]
 *   MSAQ_PRO_SILU_MUL     y = W bf16(silu(x[:, :K]) * x[:, K:])        x [M][2K]
 *   MSAQ_PRO_ADD_RMSNORM  h_out = bf16(x + addend); y = W bf16(rmsnorm(h_out, eps))
 *                         x [M][K] bf16, addend [M][K] bf16 or fp32 (addend_is_f32), h_out [M][K] bf16
 * rmsnorm(v) = v * rsqrt(mean(v^2) + eps), no gain vector.  Each intermediate is rounded to bf16 exactly as the
 * separate entry points msaq_rmsnorm / msaq_silu_mul / msaq_add_residual round it.  Column-major planes, any
 * (u, gs); formats outside the tuned path run the glue as separate kernels into the workspace tail.
 * h_out must not overlap x or addend (MSAQ_ERR_ARG): there is no in-place residual update.
 * A non-finite activation (Inf or NaN) turns its whole output row into NaN.
 */
#define MSAQ_PRO_NONE 0
#define MSAQ_PRO_RMSNORM 1
#define MSAQ_PRO_SILU_MUL 2
#define MSAQ_PRO_ADD_RMSNORM 3
size_t msaq_wonly_gemv_fused_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs);
int msaq_wonly_gemv_fused(const void* x, int prologue, const void* addend, int addend_is_f32, float eps,
                          void* h_out, const int8_t* scale_exp, const uint8_t* upper_cm,
                          const uint8_t* shared_cm, void* y, float* y_f32,
                          int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * The wide GEMV for callers that may not allocate device memory: a plugin running under a
 * host whose memory pool it must not touch, a real-time or safety-reviewed loop where
 * cudaMalloc is forbidden after start-up, a library entered from a context that owns no
 * allocator.  Same result as msaq_wonly_gemv_wide, but the split-K scratch (staged
 * activations, partial sums, counters) is a fixed array of MSAQ_STATIC_SCRATCH_BYTES inside
 * the library image; every GPU that loads the library holds that array until the process
 * exits.  The call allocates nothing and calls no allocating routine.
 *   - The first call on each device looks the array's device address up (one host-side query,
 *     no allocation); make that first call before starting a stream capture.
 *   - All calls on one device share the array and it keeps the previous call's contents: the
 *     kernels reset the words that must start at zero, but two calls that overlap on the GPU
 *     (different streams, or graphs replayed concurrently) race on it.  Serialise them.
 *   - A problem whose scratch need (msaq_wonly_gemv_workspace(1, OUT, NB, u, gs)) exceeds the
 *     array is refused with MSAQ_ERR_WORKSPACE; nothing is launched.
 * This entry point has no counterpart in the reference.
 */
#define MSAQ_STATIC_SCRATCH_BYTES (8u << 20)
size_t msaq_static_scratch_bytes(void);
int msaq_wonly_gemv_wide_static(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm,
                                const uint8_t* shared_cm, void* y, float* y_f32,
                                int64_t OUT, int64_t NB, int u, int gs, void* stream);

/* -------------------------------------------------------- KV cache write -- */

/*
 * Quantise one new token X[H,D] (bf16) into slot `pos` of the cache planes
 * (key stride Lcap), in place.  Replaces op `msaq::kv_append`
 * (csrc/pybind.cpp:236-237, host csrc/kv_attention.cu:2326-2339).
 */
int msaq_kv_append(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                   int64_t H, int64_t D, int64_t NB, int64_t pos, int64_t Lcap,
                   int u, int gs, void* stream);

/*
 * Same, after rotating each head row by the orthonormal Hadamard matrix H_D:
 * an fp32 butterfly (stages h = 1,2,..,D/2; lo' = lo+hi, hi' = lo-hi) times
 * float(1/sqrt(D)).  Replaces op `msaq::kv_append_rot`
 * (csrc/pybind.cpp:238-239, host csrc/kv_attention.cu:2343-2356).
 */
int msaq_kv_append_rot(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                       int64_t H, int64_t D, int64_t NB, int64_t pos, int64_t Lcap,
                       int u, int gs, void* stream);

/*
 * Batched append with one position per sequence: X[B*Hkv,D]; row r belongs to
 * sequence r / Hkv and is written at slot pos[r / Hkv] (int32, device memory).
 * rotate != 0 applies the Hadamard rotation first.  The reference has one
 * scalar position for the whole batch (csrc/kv_attention.cu:2326-2328); this
 * is the per-sequence form of the same two ops.
 */
int msaq_kv_append_varlen(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                          int64_t B, int64_t Hkv, int64_t D, int64_t NB, const int32_t* pos,
                          int64_t Lcap, int u, int gs, int rotate, void* stream);

/*
 * K and V rows of one decode step in one launch (no reference counterpart: the reference issues kv_append_rot for
 * K and kv_append for V, tests/harness_batchsweep.py:170-180).  Xk, Xv [B*Hkv][D] bf16; planes [B*Hkv][NB][Lcap][*];
 * slot `pos` for every sequence, or pos_per_seq[b] when that pointer is given; K is rotated when rotate_k != 0.
 * Bytes written are those of msaq_kv_append_rot / msaq_kv_append.
 */
int msaq_kv_append_pair(const void* Xk, const void* Xv, int8_t* k_scale_exp, uint8_t* k_upper, uint8_t* k_shared,
                        int8_t* v_scale_exp, uint8_t* v_upper, uint8_t* v_shared,
                        int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos, const int32_t* pos_per_seq,
                        int64_t Lcap, int u, int gs, int rotate_k, void* stream);

/*
 * Rotary position embedding fused into the cache writers and the decode prologue (no reference counterpart as an
 * operator: the reference's harness applies RoPE to q and k in PyTorch between the QKV projection and the append,
 * tests/harness_batchsweep.py:118-137 `rope_pos` / `rope_bthd`, :237).  Tables are the harness's: rope_cos / rope_sin
 * fp32 [rope_rows][D/2] in device memory with cos(pos * theta^(-2j/D)); rope_rows == 1 holds the one position of this
 * step (`rope_pos`), otherwise the row index is the token's position (`rope_tables`) and rope_rows must cover every
 * position that can occur (the capacity, for positions read from device memory).  A pair (x[2j], x[2j+1]) becomes
 * bf16(x1*c - x2*s), bf16(x1*s + x2*c) with every fp32 product and sum rounded separately, bit for bit what
 * rope_bthd yields; then the Hadamard rotation (when asked) and the quantiser see those bf16 values.
 *   msaq_rope                    out[B,heads,D] = RoPE(x[B,heads,D]) at position pos (pos_per_seq[b] when given)
 *   msaq_kv_append_pair_rope     msaq_kv_append_pair with RoPE on the K rows at the slot each row goes to
 *   msaq_kv_write_rope           msaq_kv_write with RoPE on every row at its slot (the prefill K path)
 *   msaq_kv_decode_attention_rope  the batched decode with RoPE on each query row at q_pos (q_pos_per_seq[b])
 * rope_cos == NULL turns each of the last three into the entry point it extends.
 */
int msaq_rope(const void* x, void* out, int64_t B, int64_t heads, int64_t D, const float* rope_cos,
              const float* rope_sin, int64_t rope_rows, int64_t pos, const int32_t* pos_per_seq, void* stream);
int msaq_kv_append_pair_rope(const void* Xk, const void* Xv, int8_t* k_scale_exp, uint8_t* k_upper, uint8_t* k_shared,
                             int8_t* v_scale_exp, uint8_t* v_upper, uint8_t* v_shared,
                             int64_t B, int64_t Hkv, int64_t D, int64_t NB, int64_t pos, const int32_t* pos_per_seq,
                             int64_t Lcap, int u, int gs, int rotate_k,
                             const float* rope_cos, const float* rope_sin, int64_t rope_rows, void* stream);
int msaq_kv_write_rope(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                       int64_t H, int64_t L, int64_t D, int64_t NB, int64_t key0, int64_t Lcap,
                       int u, int gs, int rotate,
                       const float* rope_cos, const float* rope_sin, int64_t rope_rows, void* stream);

/*
 * Prefill pack: X[H,L,D] (bf16) -> slots [key0, key0+L) of planes with key
 * stride Lcap (Lcap = L, key0 = 0 gives the reference's freshly allocated
 * planes).  rotate != 0 applies the Hadamard rotation to every row first.
 * Replaces op `msaq::kv_write` (csrc/pybind.cpp:235, host
 * csrc/kv_attention.cu:2302-2321).
 */
int msaq_kv_write(const void* X, int8_t* scale_exp, uint8_t* upper, uint8_t* shared,
                  int64_t H, int64_t L, int64_t D, int64_t NB, int64_t key0, int64_t Lcap,
                  int u, int gs, int rotate, void* stream);

/*
 * out[N,D] = bf16( H_D-rotation of x[N,D] ), bf16 in and out.
 * Replaces op `msaq::hadamard_rotate` (csrc/pybind.cpp:286, csrc/rotate.cu:40-86).
 */
int msaq_hadamard_rotate(const void* x, void* out, int64_t N, int64_t D, void* stream);

/*
 * Offline weight packing on the device: W[OUT,K] (bf16 if w_is_bf16 else fp32)
 * -> all five planes.  Any of the plane pointers may be NULL to skip it.
 * Device twin of ms_lib/pack.py:101-137 (`pack_weight`).
 */
int msaq_pack_weight(const void* W, int w_is_bf16, int8_t* scale_exp, uint8_t* upper,
                     uint8_t* shared, uint8_t* upper_cm, uint8_t* shared_cm,
                     int64_t OUT, int64_t K, int u, int gs, void* stream);

/* ------------------------------------------------------ KV flash-decode -- */

/* Bytes of workspace the decode entry points need (split-KV partials). */
size_t msaq_kv_decode_workspace(int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D);

/*
 * Single-sequence decode attention: q[H,D] bf16 -> out[H,D] bf16;
 * out[h] = softmax(q[h].K^T / sqrt(D)) . V over keys [0,Lk) of kv head
 * h / (H/Hkv).  Never rotates q.  Replaces op `msaq::kv_decode_attention`
 * (csrc/pybind.cpp:266-269, host csrc/kv_attention.cu:1875-2049).
 */
int msaq_kv_decode_attention(const void* q,
                             const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                             const int8_t* vs, const uint8_t* vu, const uint8_t* vh,
                             void* out, float* out_f32,
                             int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB,
                             int u, int gs, int64_t Lcap,
                             void* workspace, size_t workspace_bytes, void* stream);

/*
 * Batched decode attention: q[B,H,D], planes [B,Hkv,NB,Lcap,*] -> out[B,H,D].
 * qrot != 0 rotates each query row by H_D in the prologue (the op reads this
 * from the MS_KV_QROT environment variable, csrc/kv_attention.cu:2082-2083).
 * seq_lens (optional int32[B], device) gives per-sequence key counts <= Lk;
 * NULL means every sequence attends Lk keys, as in the reference.
 * Replaces op `msaq::kv_decode_attention_batched` (csrc/pybind.cpp:270-273,
 * host csrc/kv_attention.cu:2055-2122).
 */
int msaq_kv_decode_attention_batched(const void* q,
                                     const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                                     const int8_t* vs, const uint8_t* vu, const uint8_t* vh,
                                     void* out, float* out_f32, const int32_t* seq_lens,
                                     int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D,
                                     int64_t NB, int u, int gs, int64_t Lcap, int qrot,
                                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * One decode step's cache update and attention in one call: msaq_kv_append_pair_rope(k_new, v_new, ..., pos) followed
 * by msaq_kv_decode_attention_rope(q, ..., q_pos = pos), with the same bytes in the cache and the same output.  On
 * the tuned path (u = 4, gs = 2, D = 128, Hq/Hkv in {1,2,4,8}, Lcap % 16 == 0) the new token is packed by the
 * attention kernel itself -- the thread block that owns the key tile of the token's slot writes the K and V rows of
 * its (sequence, kv head) before it streams them -- so the append costs no launch; otherwise the two kernels run one
 * after the other.  k_new, v_new bf16 [B, Hkv, D]; pos (pos_per_seq[b] when given) is the token's slot and its
 * position for RoPE (query and K rows alike: the token attends from where it is stored); rotate_k applies the
 * Hadamard rotation to the K row; rope_cos == NULL: no RoPE.
 */
int msaq_kv_decode_attention_append(const void* q, const void* k_new, const void* v_new,
                                    int8_t* ks, uint8_t* ku, uint8_t* kh, int8_t* vs, uint8_t* vu, uint8_t* vh,
                                    void* out, float* out_f32, const int32_t* seq_lens,
                                    int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB,
                                    int u, int gs, int64_t Lcap, int rotate_k, int qrot,
                                    const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                    int64_t pos, const int32_t* pos_per_seq,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* The batched decode with the rotary embedding of the query rows in the prologue (see msaq_rope above). */
int msaq_kv_decode_attention_rope(const void* q,
                                  const int8_t* ks, const uint8_t* ku, const uint8_t* kh,
                                  const int8_t* vs, const uint8_t* vu, const uint8_t* vh,
                                  void* out, float* out_f32, const int32_t* seq_lens,
                                  int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D,
                                  int64_t NB, int u, int gs, int64_t Lcap, int qrot,
                                  const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                                  int64_t q_pos, const int32_t* q_pos_per_seq,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------- tensor-parallel exchange -- */

/*
 * out[n] = sum over ranks of partial[n] (fp32, summed in rank order: the same bits on every rank); with `residual`
 * (bf16 [n]) the result is bf16(residual + sum) instead.  No reference counterpart (the reference has no multi-GPU
 * code): this is the all-reduce of the row-parallel O and down projections of a tensor-parallel decode layer,
 * [B, hidden] fp32 per rank, done as one push over NVLink peer memory: plain peer stores of the partial sums into
 * every peer's buffer as 16-byte words that carry the exchange's sequence number beside the data, and one bounded
 * wait of every thread on its own words (no fence, no flag, no barrier between thread blocks).
 *   peer_bufs[r]  rank r's exchange memory as mapped into THIS process (world pointers, host array); every rank
 *                 allocates msaq_peer_exchange_bytes(world, n) bytes of peer-accessible memory, zero-filled once,
 *                 and exchanges the mappings (torch.distributed._symmetric_memory does both)
 *   parity        0, 1, 0, 1, ... over the successive exchanges of a process (every rank the same sequence)
 * All ranks must call it the same number of times with the same n.  A rank whose peers do not arrive within the
 * poll limit (MSAQ_OPT_WAIT_POLLS) writes NaN and sets MSAQ_STATUS_PEER_TIMEOUT; it never hangs.
 * partial == NULL: the partial sums are in the slots already -- msaq_wonly_gemv_fused_push put them there -- and the
 * call only waits, adds and writes.
 */
size_t msaq_peer_exchange_bytes(int world, int64_t n);
int msaq_peer_exchange(const float* partial, const void* residual, void* out, void* const* peer_bufs, int rank, int world,
                       int64_t n, int parity, void* stream);

/*
 * y = bf16(residual + bf16(W . pro(x))): msaq_wonly_gemv_fused (prologue none, rmsnorm or SiLU*mul) with the
 * residual add of a decoder layer's last projection done by the GEMV's finishing warps -- the same two roundings
 * as the GEMV followed by msaq_add_residual, one launch fewer.  residual and y bf16 [M, OUT]; y may be the
 * residual's own memory (every output is read before it is written, by the same thread).  Formats and sizes the
 * integer-MMA kernel does not serve run the two steps as separate kernels.
 */
int msaq_wonly_gemv_fused_add(const void* x, int prologue, float eps, const int8_t* scale_exp,
                              const uint8_t* upper_cm, const uint8_t* shared_cm, const void* residual, void* y,
                              int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                              void* workspace, size_t workspace_bytes, void* stream);

/*
 * msaq_wonly_gemv_fused with the exchange's push inside, for the row-parallel projections (O, down) of a
 * tensor-parallel layer: the warp that finishes a tile of outputs stores them straight into this rank's slot of
 * every rank's exchange buffer (its own included) instead of into local memory, so the partial sums cross NVLink
 * tile by tile while the GEMV still runs; msaq_peer_exchange(partial = NULL, ...) with the same parity and
 * n = M * OUT then completes the sum.  Same arguments as msaq_wonly_gemv_fused without y / y_f32, same peer buffers
 * and parity rule as msaq_peer_exchange.  Built into the integer-MMA kernel only (u = 4, gs = 2, M <= 8, aligned
 * column-major planes, M * OUT a multiple of 4): MSAQ_ERR_UNSUPPORTED otherwise, and the caller runs the two calls
 * separately.
 */
int msaq_wonly_gemv_fused_push(const void* x, int prologue, const void* addend, int addend_is_f32, float eps,
                               void* h_out, const int8_t* scale_exp, const uint8_t* upper_cm,
                               const uint8_t* shared_cm, int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                               void* const* peer_bufs, int rank, int world, int parity,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------- W+A decode, prefill vehicle -- */

/*
 * Run-time activation quantiser: X[M,K] bf16 -> qX int8 [M,K], the MSAQ-signed words q = up*2^u + sh of each
 * 32-block in the weights' own (u, gs) format, and sa_exp int8 [M,K/32], the block exponents; x ~ q * 2^sa_exp.
 * Bit-exact with ms_lib/reference.py:38-52 `quant_act(share=True)`.  Replaces op `msaq::quant_act`
 * (csrc/pybind.cpp:233, kernel csrc/wa_gemm.cu:82-108).
 */
int msaq_quant_act(const void* X, int8_t* qX, int8_t* sa_exp, int64_t M, int64_t K, int u, int gs, void* stream);

/*
 * W+A decode GEMV: Y[M,OUT] = sum over 32-blocks of 2^(sa+sw) * intdot(quant_act(X), q(W)), the reference's
 * `wa_matmul(share_act=True)` (ms_lib/reference.py:55-60); column-major planes, any (u, gs), any M >= 1.
 * Replaces ops `msaq::wa_gemv` (csrc/pybind.cpp:203-204) and `msaq::wa_gemv_batched` (:231-232; kernels
 * csrc/w_gemv.cu:846-1098).  The quantised activations are exact bf16 values, so after the quantiser the
 * weight-only kernels compute exactly this sum.
 */
size_t msaq_wa_gemv_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs);
int msaq_wa_gemv(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm, const uint8_t* shared_cm,
                 void* y, float* y_f32, int64_t OUT, int64_t NB, int u, int gs,
                 void* workspace, size_t workspace_bytes, void* stream);
int msaq_wa_gemv_batched(const void* X, const int8_t* scale_exp, const uint8_t* upper_cm, const uint8_t* shared_cm,
                         void* Y, float* Y_f32, int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * One-off dequantisation of a packed weight to bf16, Wbf[K,OUT] = bf16(dequant(W))^T, the operand the reference's
 * prefill hands to a dense GEMM (X[M,K] @ Wbf).  Replaces op `msaq::ms_dequant_bf16` (csrc/pybind.cpp:244-245,
 * kernel csrc/w_gemv.cu:1242-1275).
 */
int msaq_dequant_bf16(const int8_t* scale_exp, const uint8_t* upper_cm, const uint8_t* shared_cm, void* Wbf,
                      int64_t OUT, int64_t K, int u, int gs, void* stream);

/* ------------------------------------------------- plain MXINT8 baseline -- */

/*
 * The reference's matched baseline format (ms_lib/pack.py:530-594: one int8 code per element on the block grid
 * 2^e, e the same block exponent as MSAQ; 33 bytes per 32 values): the reference's headline metric is the time of
 * an MSAQ kernel over the time of its MXINT8 twin at the same optimisation level (methodology.md:34-38), so the
 * twins here run the same pipelines as the tuned MSAQ kernels with the sub-byte decode taken out.
 *   weights   scale_exp int8 [nb,OUT]   qweight int8 [nb,32,OUT]   qweight_cm int8 [nb,OUT,32]
 *   KV cache  scale_exp int8 [B*Hkv,nb,Lcap]   qweight int8 [B*Hkv,nb,Lcap,32]
 * msaq_mxint8_pack_weight      device twin of pack_weight_mxint8 (ms_lib/pack.py:546-566); any plane may be NULL
 * msaq_mxint8_gemv_wide        replaces op `msaq::mxint8_gemv_wide` (csrc/pybind.cpp:290-291, csrc/mxint8.cu:196-253)
 * msaq_mxint8_gemv_batched_wide  replaces op `msaq::mxint8_gemv_batched_wide` (csrc/pybind.cpp:292-293); any M >= 1,
 *                              OUT a multiple of 16
 * msaq_mxint8_kv_append        replaces op `msaq::mxint8_kv_append` (csrc/pybind.cpp:321-322)
 * msaq_mxint8_kv_write         replaces op `msaq::mxint8_kv_write` (csrc/pybind.cpp:320), into slots [key0, key0+L)
 * msaq_mxint8_kv_decode_batched  replaces ops `msaq::mxint8_kv_decode[_batched]` (csrc/pybind.cpp:314-319); optional
 *                              per-sequence lengths; head_dim 128, Hq/Hkv in {1,2,4,8}, Lcap a multiple of 16
 *                              (workspace: msaq_kv_decode_workspace)
 */
int msaq_mxint8_pack_weight(const void* W, int w_is_bf16, int8_t* scale_exp, int8_t* qweight, int8_t* qweight_cm,
                            int64_t OUT, int64_t K, void* stream);
size_t msaq_mxint8_gemv_workspace(int64_t M, int64_t OUT, int64_t NB);
int msaq_mxint8_gemv_wide(const void* x, const int8_t* scale_exp, const int8_t* qweight_cm, void* y, float* y_f32,
                          int64_t OUT, int64_t NB, void* workspace, size_t workspace_bytes, void* stream);
int msaq_mxint8_gemv_batched_wide(const void* X, const int8_t* scale_exp, const int8_t* qweight_cm, void* Y, float* Y_f32,
                                  int64_t M, int64_t OUT, int64_t NB, void* workspace, size_t workspace_bytes,
                                  void* stream);
int msaq_mxint8_kv_append(const void* X, int8_t* scale_exp, int8_t* qweight, int64_t H, int64_t D, int64_t NB,
                          int64_t pos, int64_t Lcap, void* stream);
int msaq_mxint8_kv_write(const void* X, int8_t* scale_exp, int8_t* qweight, int64_t H, int64_t L, int64_t D, int64_t NB,
                         int64_t key0, int64_t Lcap, void* stream);
int msaq_mxint8_kv_decode_batched(const void* q, const int8_t* ks, const int8_t* kq, const int8_t* vs, const int8_t* vq,
                                  void* out, float* out_f32, const int32_t* seq_lens,
                                  int64_t B, int64_t H, int64_t Hkv, int64_t Lk, int64_t D, int64_t NB, int64_t Lcap,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------- layer-step glue -- */

/*
 * Fused element-wise steps between the packed GEMVs of a decoder-layer decode step; the
 * reference leaves them to PyTorch (tests/harness_batchsweep.py:230-243) and has no op for them.
 *   msaq_rmsnorm      out[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps)          bf16 in/out, fp32 math
 *   msaq_silu_mul     out[r,j] = silu(gate_up[r,j]) * gate_up[r,F+j]           bf16 in/out
 *   msaq_add_residual out = bf16(h + delta), delta fp32 (delta_is_f32 != 0) or bf16
 */
int msaq_rmsnorm(const void* x, void* out, int64_t rows, int64_t n, float eps, void* stream);
int msaq_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t F, void* stream);
int msaq_add_residual(const void* h, const void* delta, int delta_is_f32, void* out, int64_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MSAQ_B200_H */
