// context.cu -- part 1 of the C ABI: the device layer behind the reference's PROVE
// (src/sumcheck.lisp:512-571).  A context owns the tables, the ping-pong buffers of the folded
// tables, the eq weights of every round and the buffers of the partial sums, and runs one round
// kernel per sc_round.  The transcript stays with the caller: per round POINTS * D words go to
// the host and D words come back.
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "device.h"

using namespace sc;
using namespace scf;

// ------------------------------------------------------------------ NCCL, loaded on first use
// Only the multi-GPU path needs it, so the library carries no link-time dependency on it.
namespace {
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { NCCL_UINT32 = 3 };
struct Nccl {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool load() {
        if (handle) return true;
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *nm : names) {
            handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
            if (handle) break;
        }
        if (!handle) return false;
        GetUniqueId = (decltype(GetUniqueId))dlsym(handle, "ncclGetUniqueId");
        CommInitRank = (decltype(CommInitRank))dlsym(handle, "ncclCommInitRank");
        CommDestroy = (decltype(CommDestroy))dlsym(handle, "ncclCommDestroy");
        CommAbort = (decltype(CommAbort))dlsym(handle, "ncclCommAbort");
        AllGather = (decltype(AllGather))dlsym(handle, "ncclAllGather");
        GetErrorString = (decltype(GetErrorString))dlsym(handle, "ncclGetErrorString");
        return GetUniqueId && CommInitRank && CommDestroy && CommAbort && AllGather && GetErrorString;
    }
} g_nccl;
}  // namespace

// ------------------------------------------------------------------ the context

struct TableState {
    u32 *t0 = nullptr;          // the caller's table on the device (canonical words)
    u64 t0_cap = 0;             // bytes allocated
    bool borrowed = false;      // t0 is the caller's device memory (sc_borrow_table): never freed or written here
    u64 entries = 0;
    int stride = 0;
    u32 *buf[2] = {nullptr, nullptr};   // ping-pong buffers of the folded table (D canonical words per entry)
    u64 buf_cap[2] = {0, 0};
    // the table as the next kernel reads it
    const u32 *cur = nullptr;
    int cur_buf = -1;           // -1: t0 (or the gathered buffer), else buf index
    bool cur_base = false;
    u64 cur_entries = 0;
};

struct RoundPlan {
    int logL = 0;
    bool use_low = false, use_high = false;
    u64 low_word = 0, high_word = 0;
};

struct sc_ctx {
    int device = 0;
    int sms = 148;
    int blocks_per_sm = 2;           // round-kernel blocks launched per SM (SABLE_B200_BLOCKS_PER_SM overrides)
    bool force_generic = false;      // SABLE_B200_GENERIC at sc_create: every statement runs the term-table kernel
    cudaStream_t stream = nullptr;
    std::string last_error;
    u64 budget = 0, used = 0;
    uint64_t launches = 0;

    // statement
    int D = 0, points = 0, ntables = 0, nt_used = 0;
    bool have_statement = false;
    int order[SC_MAX_TABLES];        // kernel position -> slot (the statement's tables first)
    DevStatement st;                 // factors are kernel positions

    TableState tab[SC_MAX_TABLES];

    // proof state
    bool begun = false, have_r = false, have_eq = false;
    int n = 0, K = 1, j = 0;
    int nloc = 0;                    // variables of a rank's slice (n - log2 world)
    int gather_round = 0;            // the round before which the slices are gathered: every rank then holds the
                                     // whole (small) tables and the rounds need no exchange any more
    u32 r[8];
    u32 post[8];                     // the final factor of a round: R^e of the statement times this rank's eq weight
    bool use_post = false;
    int st_e = 0;                    // e of the statement (see DevTerm)
    u32 st_re = 0;                   // R^e in Montgomery form
    u32 seq = 0;                     // number of the last round launch; the kernel posts it after the sums
    bool sv_statement = false;       // the statement can take the small-value rounds: base-field coefficients, few short terms
    int base_groups = 0;             // > 0: the statement can run the base-table kernel with this many groups
    u32 gcoef[2][8];                 // the groups' coefficients (Montgomery form)
    int shape = SHAPE_GENERIC;       // the kernel family of the statement
    u32 st_factor[8];                // a product statement's coefficient (canonical), applied with the final factor
    bool use_factor = false;
    std::vector<RoundPlan> plan;

    // device buffers
    u32 *d_eq = nullptr, *d_bw = nullptr, *d_chunks = nullptr, *d_weights = nullptr;
    u64 eq_cap = 0, bw_cap = 0, chunks_cap = 0, weights_cap = 0;
    WeightDesc *d_descs = nullptr;
    u64 descs_cap = 0;
    std::vector<u32> stage_eq, stage_bw;          // what sc_begin copies to the device, kept alive past the call
    std::vector<WeightDesc> stage_descs;
    u32 *d_partials = nullptr;
    unsigned int *d_counter = nullptr;
    u32 *d_out = nullptr, *h_out = nullptr, *h_out_dev = nullptr;   // h_out: mapped pinned; h_out_dev its device alias
    u32 *d_export = nullptr, *h_export = nullptr;
    u64 export_cap = 0;
    std::vector<sc_ctx *> children;  // contexts of this one's own on the same device (sc_child), destroyed with it
    void *d_work = nullptr;          // a caller's scratch (sc_workspace), grow-only
    u64 work_cap = 0;
    u32 *d_gather = nullptr;         // world * SV_MAX_WORDS words: the ranks' sums side by side
    u32 *d_sv = nullptr;             // this rank's small-value accumulators
    u32 *d_gtab[SC_MAX_TABLES];      // gathered tables
    u64 gtab_cap[SC_MAX_TABLES] = {0};
    int grid_cap = 0;

    // the resident kernel of the last rounds (see TailArgs)
    u32 *h_tail = nullptr, *h_tail_dev = nullptr;   // mapped host memory and its device alias
    bool tail_active = false;
    int tail_first = 0, tail_rounds = 0, tail_nofold = 0, tail_bits = 12;
    u32 tail_seq = 0;
    unsigned tail_polls = TAIL_POLL_LIMIT;
    u64 tail_entries = 0;            // entries of the tables the first round of the launch read
    int tail_buf0[SC_MAX_TABLES];    // per slot: which of the table's two buffers the first round wrote
    const sc_transcript *attached = nullptr;   // the host transcript a chain copies its hash state from
    bool tail_own = false;           // the running resident kernel derives its challenges itself

    // the transcript on the device: every round of a proof enqueued at once, each launch's last block sending its
    // sums and drawing the challenge the next launch folds by (see RoundArgs::tstate)
    bool device_transcript = false;  // SABLE_B200_DEVICE_TRANSCRIPT=1 at sc_create, or sc_set_device_transcript
    u32 *d_tstate = nullptr;         // the hash state between launches, B3_STATE_WORDS words
    u32 *d_chal = nullptr;           // per round 16 words: the challenge in Montgomery form, then canonical
    u32 *h_chain = nullptr, *h_chain_dev = nullptr;   // mapped host memory: per round CHAIN_SLOT_WORDS words
    bool chain_active = false;
    int chain_first = 0;             // the first round of the chain
    int chain_end = 0;               // the first round not run by a round kernel of the chain: the resident kernel's first, or n
    u32 chain_seq = 0;               // round j of the chain posts chain_seq + j
    bool have_state = false;         // a hash state handed over by sc_attach_transcript_state, not used yet
    u32 state0[B3_STATE_WORDS];
    std::chrono::steady_clock::time_point chain_t0;   // when the chain's last launch was enqueued (for SABLE_B200_TRACE)

    // the first two rounds from one pass over base tables (see SvArgs)
    bool sv_ok = false;
    int sv_l0 = 2;                   // the rounds answered from the accumulators: 2, or 3 (degree at most two)
    u32 sv_A[SV3_MAX_WORDS];         // the accumulators, canonical: G^l0 elements, index sum z_t G^t
    u32 sv_rho[3][8];                // the challenges of those rounds
    u32 sv_eq[3][8];                 // eq elements 1 and 2, canonical (the weights of the variables still open in those rounds' messages)
    u32 *h_sv = nullptr, *h_sv_dev = nullptr;

    // timing
    bool timing = false;
    std::vector<cudaEvent_t> ev;
    std::vector<sc_round_stat> stats;

    // communicator
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, logw = 0;
    // mailboxes for the exchange of the round sums by peer stores (see RoundArgs::mail)
    u32 *mail[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    bool p2p = false;
    u32 xseq = 0;
    int comm_timeout_s = 30;         // a round whose exchange has not finished after this long aborts the communicator
    unsigned mail_polls = MAIL_POLL_LIMIT;   // polls a round kernel's last block waits for the other ranks' sums (SABLE_B200_MAIL_POLLS)
};

constexpr int CHAIN_MAX_ROUNDS = 64;

static int fail(sc_ctx *c, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (c) c->last_error = buf;
    return code;
}
#define CU(call)                                                                                          \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess) return fail(ctx, e_ == cudaErrorMemoryAllocation ? SC_ENOMEM : SC_ECUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

static int dev_alloc(sc_ctx *ctx, void **p, u64 bytes) {
    if (ctx->budget && ctx->used + bytes > ctx->budget)
        return fail(ctx, SC_ENOMEM, "memory budget: %llu bytes held, %llu more asked, cap %llu", (unsigned long long)ctx->used,
                    (unsigned long long)bytes, (unsigned long long)ctx->budget);
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(ctx, SC_ENOMEM, "cudaMalloc of %llu bytes: %s", (unsigned long long)bytes, cudaGetErrorString(e)); }
    ctx->used += bytes;
    return SC_OK;
}
static void dev_free(sc_ctx *ctx, void *p, u64 bytes) {
    if (!p) return;
    cudaFree(p);
    ctx->used -= bytes <= ctx->used ? bytes : ctx->used;
}
// grow a buffer to at least BYTES (contents are not kept)
template <class T> static int ensure(sc_ctx *ctx, T **p, u64 *cap, u64 bytes) {
    if (*p && *cap >= bytes) return SC_OK;
    dev_free(ctx, *p, *cap);
    *p = nullptr; *cap = 0;
    int rc = dev_alloc(ctx, (void **)p, bytes);
    if (rc) return rc;
    *cap = bytes;
    return SC_OK;
}

// Make the resident kernel of the last rounds return (it polls this word), and wait for it.
static void tail_stop(sc_ctx *ctx) {
    ctx->chain_active = false;   // a chain's launches wait for nobody: whatever follows on the stream comes after them
    if (!ctx->tail_active) return;
    *(volatile u32 *)(ctx->h_tail + TAIL_STOP) = ctx->tail_seq;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    cudaStreamSynchronize(ctx->stream);
    ctx->tail_active = false;
}

// A collective that does not finish (a rank left, a link went down) is ended from the host: the
// communicator is aborted, which makes its kernels return, and the context goes back to one GPU.
static void comm_abort(sc_ctx *ctx) {
    if (!ctx->comm) return;
    g_nccl.CommAbort(ctx->comm);
    ctx->comm = nullptr;
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < 8; r++) {
        if (!ctx->mail[r]) continue;
        if (r == ctx->rank) cudaFree(ctx->mail[r]); else cudaIpcCloseMemHandle(ctx->mail[r]);
        ctx->mail[r] = nullptr;
    }
    ctx->p2p = false;
    ctx->world = 1; ctx->rank = 0; ctx->logw = 0;
    ctx->begun = false;
}

// Wait until a word of mapped memory holds WANT.  Bounded: the stream finishing without the word
// showing, or the time limit passing, ends the wait (with a communicator, by aborting it).
static bool wait_word(sc_ctx *ctx, const u32 *word, u32 want) {
    volatile const u32 *w = word;
    const auto t0 = std::chrono::steady_clock::now();
    for (u64 spin = 0;; spin++) {
        if ((*w & ~EXCHANGE_FAILED) == want) { std::atomic_thread_fence(std::memory_order_acquire); return true; }
        if ((spin & 0xfffff) == 0xfffff) {
            if (cudaStreamQuery(ctx->stream) != cudaErrorNotReady) {
                cudaStreamSynchronize(ctx->stream);
                std::atomic_thread_fence(std::memory_order_acquire);
                return (*w & ~EXCHANGE_FAILED) == want;
            }
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(ctx->comm_timeout_s)) {
                comm_abort(ctx);
                return false;
            }
        }
    }
}

// Wait until COUNT words of mapped memory all carry the mark TAIL_HERE (each word says for itself that the device has
// written it).  Bounded like wait_word.
static bool wait_here(sc_ctx *ctx, const u32 *words, int count) {
    volatile const u32 *w = words;
    const auto t0 = std::chrono::steady_clock::now();
    for (u64 spin = 0;; spin++) {
        u32 all = TAIL_HERE;
        for (int k = 0; k < count; k++) all &= w[k];
        if (all) { std::atomic_thread_fence(std::memory_order_acquire); return true; }
        if ((spin & 0xfffff) == 0xfffff) {
            if (cudaStreamQuery(ctx->stream) != cudaErrorNotReady) {
                cudaStreamSynchronize(ctx->stream);
                std::atomic_thread_fence(std::memory_order_acquire);
                all = TAIL_HERE;
                for (int k = 0; k < count; k++) all &= w[k];
                return all != 0;
            }
            if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(ctx->comm_timeout_s)) {
                comm_abort(ctx);
                return false;
            }
        }
    }
}

extern "C" const char *sc_strerror(int code) {
    switch (code) {
    case SC_OK: return "ok";
    case SC_EINVAL: return "invalid parameter";
    case SC_ECUDA: return "CUDA error";
    case SC_ENOMEM: return "out of memory";
    case SC_EUNSUPPORTED: return "unsupported shape";
    case SC_ESTATE: return "call out of order";
    case SC_ECOMM: return "communicator error";
    case SC_ESTATEMENT: return "bad statement";
    default: return "unknown error";
    }
}
extern "C" const char *sc_last_error(const sc_ctx *ctx) { return ctx ? ctx->last_error.c_str() : ""; }

extern "C" int sc_create(int device, sc_ctx **out) {
    if (!out) return SC_EINVAL;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { cudaGetLastError(); return SC_ECUDA; }
    if (device < 0 || device >= count) return SC_EINVAL;
    sc_ctx *ctx = new sc_ctx();
    ctx->device = device;
    for (int t = 0; t < SC_MAX_TABLES; t++) ctx->d_gtab[t] = nullptr;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { delete ctx; return SC_ECUDA; }
    ctx->sms = prop.multiProcessorCount;
    if (const char *env = getenv("SABLE_B200_BLOCKS_PER_SM")) { int v = atoi(env); if (v >= 1 && v <= 8) ctx->blocks_per_sm = v; }
    ctx->force_generic = getenv("SABLE_B200_GENERIC") != nullptr;
    ctx->grid_cap = ctx->sms * 8;
    bool ok = cudaMalloc(&ctx->d_partials, (size_t)ctx->grid_cap * PARTIAL_ROW_WORDS * 4) == cudaSuccess &&
              cudaMalloc(&ctx->d_counter, 64) == cudaSuccess && cudaMemset(ctx->d_counter, 0, 64) == cudaSuccess &&
              cudaMalloc(&ctx->d_out, (MAX_PARTIAL_WORDS + 32) * 4) == cudaSuccess &&
              cudaHostAlloc(&ctx->h_out, (MAX_PARTIAL_WORDS + 32) * 4, cudaHostAllocMapped) == cudaSuccess &&
              cudaHostGetDevicePointer(&ctx->h_out_dev, ctx->h_out, 0) == cudaSuccess;
    ok = ok && cudaHostAlloc(&ctx->h_tail, TAIL_WORDS * 4, cudaHostAllocMapped) == cudaSuccess &&
         cudaHostGetDevicePointer(&ctx->h_tail_dev, ctx->h_tail, 0) == cudaSuccess;
    if (!ok) { cudaGetLastError(); sc_destroy(ctx); return SC_ECUDA; }
    memset(ctx->h_tail, 0, TAIL_WORDS * 4);
    memset(ctx->h_out, 0, (MAX_PARTIAL_WORDS + 32) * 4);   // pinned memory comes back as an earlier context left it: its posted words must not be taken for ours
    if (cudaHostAlloc(&ctx->h_sv, (SV3_MAX_WORDS + 32) * 4, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(&ctx->h_sv_dev, ctx->h_sv, 0) != cudaSuccess) { cudaGetLastError(); sc_destroy(ctx); return SC_ECUDA; }
    memset(ctx->h_sv, 0, (SV3_MAX_WORDS + 32) * 4);
    if (cudaMalloc(&ctx->d_tstate, B3_STATE_WORDS * 4) != cudaSuccess || cudaMemset(ctx->d_tstate, 0, B3_STATE_WORDS * 4) != cudaSuccess ||
        cudaMalloc(&ctx->d_chal, (size_t)CHAIN_MAX_ROUNDS * 16 * 4) != cudaSuccess ||
        cudaHostAlloc(&ctx->h_chain, (size_t)CHAIN_MAX_ROUNDS * CHAIN_SLOT_WORDS * 4, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(&ctx->h_chain_dev, ctx->h_chain, 0) != cudaSuccess) { cudaGetLastError(); sc_destroy(ctx); return SC_ECUDA; }
    memset(ctx->h_chain, 0, (size_t)CHAIN_MAX_ROUNDS * CHAIN_SLOT_WORDS * 4);
    if (const char *env = getenv("SABLE_B200_DEVICE_TRANSCRIPT")) ctx->device_transcript = env[0] == '1';
    if (const char *env = getenv("SABLE_B200_TAIL_BITS")) ctx->tail_bits = std::max(0, std::min(14, atoi(env)));
    if (const char *env = getenv("SABLE_B200_COMM_TIMEOUT_S")) ctx->comm_timeout_s = std::max(1, atoi(env));
    if (const char *env = getenv("SABLE_B200_MAIL_POLLS")) ctx->mail_polls = (unsigned)std::max(1000, std::min((int)MAIL_POLL_LIMIT, atoi(env)));
    if (const char *env = getenv("SABLE_B200_TAIL_POLLS")) ctx->tail_polls = (unsigned)std::max(1000, std::min((int)TAIL_POLL_LIMIT, atoi(env)));
    *out = ctx;
    return SC_OK;
}

extern "C" int sc_destroy(sc_ctx *ctx) {
    if (!ctx) return SC_OK;
    for (sc_ctx *c : ctx->children) sc_destroy(c);
    ctx->children.clear();
    cudaSetDevice(ctx->device);
    tail_stop(ctx);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->h_tail) cudaFreeHost(ctx->h_tail);
    if (ctx->h_sv) cudaFreeHost(ctx->h_sv);
    if (ctx->h_chain) cudaFreeHost(ctx->h_chain);
    cudaFree(ctx->d_tstate); cudaFree(ctx->d_chal);
    for (int r = 0; r < 8; r++) {
        if (!ctx->mail[r]) continue;
        if (r == ctx->rank || ctx->world == 1) cudaFree(ctx->mail[r]); else cudaIpcCloseMemHandle(ctx->mail[r]);
    }
    if (ctx->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->comm);
    for (auto &t : ctx->tab) { if (!t.borrowed) cudaFree(t.t0); cudaFree(t.buf[0]); cudaFree(t.buf[1]); }
    for (auto p : ctx->d_gtab) cudaFree(p);
    cudaFree(ctx->d_eq); cudaFree(ctx->d_bw); cudaFree(ctx->d_chunks); cudaFree(ctx->d_weights); cudaFree(ctx->d_descs);
    cudaFree(ctx->d_sv); cudaFree(ctx->d_partials); cudaFree(ctx->d_counter); cudaFree(ctx->d_out); cudaFree(ctx->d_export); cudaFree(ctx->d_gather); cudaFree(ctx->d_work);
    if (ctx->h_out) cudaFreeHost(ctx->h_out);
    if (ctx->h_export) cudaFreeHost(ctx->h_export);
    for (auto e : ctx->ev) cudaEventDestroy(e);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    cudaGetLastError();
    delete ctx;
    return SC_OK;
}

extern "C" int sc_set_memory_budget(sc_ctx *ctx, uint64_t bytes) {
    if (!ctx) return SC_EINVAL;
    ctx->budget = bytes;
    return SC_OK;
}
extern "C" uint64_t sc_launch_count(const sc_ctx *ctx) { return ctx ? ctx->launches : 0; }

extern "C" int sc_enable_timing(sc_ctx *ctx, int on) {
    if (!ctx) return SC_EINVAL;
    ctx->timing = on != 0;
    return SC_OK;
}
extern "C" int sc_round_stats(sc_ctx *ctx, sc_round_stat *stats, int cap, int *count) {
    if (!ctx || !count) return SC_EINVAL;
    *count = (int)ctx->stats.size();
    for (int i = 0; i < *count && i < cap && stats; i++) stats[i] = ctx->stats[i];
    return SC_OK;
}

extern "C" int sc_timer_start(sc_ctx *ctx) {
    if (!ctx) return SC_EINVAL;
    cudaSetDevice(ctx->device);
    while (ctx->ev.size() < 4) { cudaEvent_t e; CU(cudaEventCreate(&e)); ctx->ev.push_back(e); }
    CU(cudaEventRecord(ctx->ev[2], ctx->stream));
    return SC_OK;
}
extern "C" int sc_timer_stop(sc_ctx *ctx, float *ms) {
    if (!ctx || !ms || ctx->ev.size() < 4) return SC_EINVAL;
    cudaSetDevice(ctx->device);
    CU(cudaEventRecord(ctx->ev[3], ctx->stream));
    CU(cudaEventSynchronize(ctx->ev[3]));
    CU(cudaEventElapsedTime(ms, ctx->ev[2], ctx->ev[3]));
    return SC_OK;
}

// ------------------------------------------------------------------ statement

// a b for elements in Montgomery form, on the host
static void ext_mul_host(int D, const u32 *a, const u32 *b, u32 *o) {
    if (D == 4) {
        Ext<4> x, y; for (int c = 0; c < 4; c++) { x.v[c] = a[c]; y.v[c] = b[c]; }
        Ext<4> z = emul<4>(x, y); for (int c = 0; c < 4; c++) o[c] = z.v[c];
    } else {
        Ext<8> x, y; for (int c = 0; c < 8; c++) { x.v[c] = a[c]; y.v[c] = b[c]; }
        Ext<8> z = emul<8>(x, y); for (int c = 0; c < 8; c++) o[c] = z.v[c];
    }
}

// 1/a for a nonzero element in Montgomery form, as a^(p^D - 2) (the same element as the reference's norm
// descent, INV*, src/field.lisp:236-243); used once per statement at most
static void ext_inv_host(int D, const u32 *a, u32 *o) {
    u32 ex[9] = {1, 0, 0, 0, 0, 0, 0, 0, 0};   // p^D - 2, little-endian 32-bit words
    int len = 1;
    for (int k = 0; k < D; k++) {
        u64 carry = 0;
        for (int i = 0; i < len; i++) { const u64 t = (u64)ex[i] * P + carry; ex[i] = (u32)t; carry = t >> 32; }
        if (carry) ex[len++] = (u32)carry;
    }
    for (int i = 0, borrow = 2; i < len && borrow; i++) {
        if (ex[i] >= (u32)borrow) { ex[i] -= (u32)borrow; borrow = 0; } else { ex[i] -= (u32)borrow; borrow = 1; }
    }
    u32 r[8] = {R1, 0, 0, 0, 0, 0, 0, 0}, base[8];
    memcpy(base, a, 4 * (size_t)D);
    for (int i = 0; i < len; i++)
        for (int b = 0; b < 32; b++) {
            if ((ex[i] >> b) & 1) ext_mul_host(D, r, base, r);
            ext_mul_host(D, base, base, base);
        }
    memcpy(o, r, 4 * (size_t)D);
}

// R^k mod p for any integer k (R = 2^32)
static u32 pow_r(int k) {
    auto pw = [](u32 b, u64 ex) { u64 r = 1, x = b; for (; ex; ex >>= 1) { if (ex & 1) r = r * x % P; x = x * x % P; } return (u32)r; };
    return k >= 0 ? pw(R1, (u64)k) : pw(pw(R1, P - 2), (u64)(-k));
}

// The statements with kernels of their own (device.h): can the statement's tables be put into the entry's positions
// so that the terms' table lists agree, with no coefficient beyond the kind the entry's term takes?
static bool match_listed(const ListedInfo &L, int D, int ntables, int nterms, const uint32_t *coeffs, const int32_t *term_ptr,
                         const int32_t *term_tables, const bool *used, int *slot_at, int *term_at) {
    int slots[SC_MAX_TABLES], ns = 0;
    for (int s = 0; s < ntables; s++) if (used[s]) slots[ns++] = s;
    if (ns != L.nt || nterms != L.nterms || nterms > LISTED_MAX_TERMS) return false;
    for (int t = 0; t < nterms; t++) if (term_ptr[t + 1] - term_ptr[t] > LISTED_MAX_FACTORS) return false;
    int perm[SC_MAX_TABLES];
    for (int k = 0; k < ns; k++) perm[k] = k;
    do {   // position k holds slot slots[perm[k]]
        int pos_of[SC_MAX_TABLES] = {0};
        for (int k = 0; k < ns; k++) pos_of[slots[perm[k]]] = k;
        int torder[LISTED_MAX_TERMS] = {0, 1, 2};
        do {   // statement term t plays the entry's term torder[t]
            bool ok = true;
            for (int t = 0; t < nterms && ok; t++) {
                const int e = torder[t], nf = term_ptr[t + 1] - term_ptr[t];
                if (nf != L.nf[e]) { ok = false; break; }
                int mine[LISTED_MAX_FACTORS], theirs[LISTED_MAX_FACTORS];
                for (int k = 0; k < nf; k++) { mine[k] = pos_of[term_tables[term_ptr[t] + k]]; theirs[k] = L.f[e][k]; }
                std::sort(mine, mine + nf); std::sort(theirs, theirs + nf);
                for (int k = 0; k < nf; k++) ok = ok && mine[k] == theirs[k];
                bool upper = false;
                for (int c = 1; c < D; c++) upper = upper || coeffs[(size_t)t * D + c] % P != 0;
                if (upper && L.ck[e] != CK_EXT) ok = false;
            }
            if (ok) {
                for (int k = 0; k < ns; k++) slot_at[k] = slots[perm[k]];
                for (int t = 0; t < nterms; t++) term_at[t] = torder[t];
                return true;
            }
        } while (std::next_permutation(torder, torder + nterms));
    } while (std::next_permutation(perm, perm + ns));
    return false;
}

extern "C" int sc_set_statement(sc_ctx *ctx, int D, int points, int ntables, int nterms, const uint32_t *coeffs,
                                const int32_t *term_ptr, const int32_t *term_tables) {
    if (!ctx) return SC_EINVAL;
    tail_stop(ctx);
    if (D != 4 && D != 8) return fail(ctx, SC_EINVAL, "extension degree %d: expected 4 or 8", D);
    if (points < 1) return fail(ctx, SC_EINVAL, "points %d: expected at least 1", points);
    if (ntables < 1 || nterms < 0 || (nterms && (!coeffs || !term_ptr))) return fail(ctx, SC_EINVAL, "bad term table");
    if (ntables > SC_MAX_TABLES) return fail(ctx, SC_EUNSUPPORTED, "%d tables: at most %d", ntables, SC_MAX_TABLES);
    if (nterms > SC_MAX_TERMS) return fail(ctx, SC_EUNSUPPORTED, "%d terms: at most %d", nterms, SC_MAX_TERMS);
    if (points > SC_MAX_POINTS) return fail(ctx, SC_EUNSUPPORTED, "degree %d: at most %d", points, SC_MAX_POINTS);
    bool used[SC_MAX_TABLES] = {false};
    for (int t = 0; t < nterms; t++) {
        const int nf = term_ptr[t + 1] - term_ptr[t];
        if (nf < 0 || nf > SC_MAX_FACTORS) return fail(ctx, SC_EUNSUPPORTED, "term %d has %d factors: at most %d", t, nf, SC_MAX_FACTORS);
        for (int k = term_ptr[t]; k < term_ptr[t + 1]; k++) {
            if (term_tables[k] < 0 || term_tables[k] >= ntables) return fail(ctx, SC_EINVAL, "term %d names table %d of %d", t, term_tables[k], ntables);
            used[term_tables[k]] = true;
        }
    }
    // the statement's tables first, in slot order; the others (only folded) after them
    int pos_of[SC_MAX_TABLES], npos = 0;
    int occurrences[SC_MAX_TABLES] = {0};
    for (int t = 0; t < nterms; t++) for (int k = term_ptr[t]; k < term_ptr[t + 1]; k++) occurrences[term_tables[k]]++;
    int nt_used = 0;
    for (int s = 0; s < ntables; s++) nt_used += used[s];
    if (nt_used > 8) return fail(ctx, SC_EUNSUPPORTED, "the statement multiplies %d different tables: at most 8", nt_used);

    // statements with a kernel of their own (see Shape)
    int shape = SHAPE_GENERIC, lam_term = -1, a_term = -1, b_term = -1;
    int first[SC_MAX_TABLES];
    int nfirst = 0;
    auto same_coefficient = [&](int t, int u) {
        bool nonzero = false;
        for (int c = 0; c < D; c++) {
            if (coeffs[(size_t)t * D + c] % P != coeffs[(size_t)u * D + c] % P) return false;
            nonzero = nonzero || coeffs[(size_t)t * D + c] % P != 0;
        }
        return nonzero;
    };
    auto is_one = [&](int t) {
        for (int c = 0; c < D; c++) if (coeffs[(size_t)t * D + c] % P != (c == 0 ? 1u : 0u)) return false;
        return true;
    };
    if (nterms == 1 && term_ptr[1] - term_ptr[0] == nt_used && points == nt_used && nt_used >= 1) {
        bool distinct = true;
        for (int s = 0; s < ntables; s++) if (occurrences[s] > 1) distinct = false;
        if (distinct) shape = SHAPE_PRODUCT;
    } else if (nterms == 3 && nt_used == 4 && points == 2) {
        // a d + b c + lam c d: two tables occur twice (c, d) and share the term with the free coefficient
        int doubles[4], nd = 0;
        bool ok = true;
        for (int s = 0; s < ntables; s++) { if (occurrences[s] == 2) doubles[nd++ & 3] = s; else if (occurrences[s] > 2) ok = false; }
        for (int t = 0; t < 3; t++) if (term_ptr[t + 1] - term_ptr[t] != 2) ok = false;
        if (ok && nd == 2) {
            const int c = doubles[0], d = doubles[1];
            int a = -1, b = -1;
            for (int t = 0; t < 3; t++) {
                const int x = term_tables[term_ptr[t]], y = term_tables[term_ptr[t] + 1];
                if ((x == c && y == d) || (x == d && y == c)) lam_term = t;
                else if (x == d || y == d) { a = (x == d) ? y : x; a_term = t; }
                else if (x == c || y == c) { b = (x == c) ? y : x; b_term = t; }
            }
            // the two single products must carry one and the same coefficient: it is taken out in front
            // (reference LAYER-STATEMENT: a (p0 q1 + p1 q0) + (a lambda) q0 q1, src/gkr.lisp:30-41)
            if (lam_term >= 0 && a >= 0 && b >= 0 && a != b && occurrences[a] == 1 && occurrences[b] == 1 &&
                same_coefficient(a_term, b_term)) {
                shape = SHAPE_GKR;
                first[0] = a; first[1] = b; first[2] = c; first[3] = d; nfirst = 4;
            }
        }
    }
    int term_at[SC_MAX_TERMS];
    for (int t = 0; t < SC_MAX_TERMS; t++) term_at[t] = t;
    const ListedInfo *listed_match = nullptr;
    if (shape == SHAPE_GENERIC && nterms >= 1 && !ctx->force_generic) {
        static const ListedInfo listed[LISTED_SHAPES] = {listed_info<0>(), listed_info<1>(), listed_info<2>()};
        for (int k = 0; k < LISTED_SHAPES; k++)
            if (points == listed[k].pts && match_listed(listed[k], D, ntables, nterms, coeffs, term_ptr, term_tables, used, first, term_at)) {
                shape = SHAPE_LISTED + k;
                nfirst = listed[k].nt;
                listed_match = &listed[k];
                break;
            }
    }
    bool placed[SC_MAX_TABLES] = {false};
    for (int k = 0; k < nfirst; k++) { ctx->order[npos] = first[k]; pos_of[first[k]] = npos++; placed[first[k]] = true; }
    for (int s = 0; s < ntables; s++) if (used[s] && !placed[s]) { ctx->order[npos] = s; pos_of[s] = npos++; placed[s] = true; }
    for (int s = 0; s < ntables; s++) if (!placed[s]) { ctx->order[npos] = s; pos_of[s] = npos++; }
    if (!round_supported(D, points, nt_used > 0 ? nt_used : 1))
        return fail(ctx, SC_EUNSUPPORTED, "no kernel for degree %d over %d tables (degree above 4: at most 4 tables)", points, nt_used);
    if (ctx->force_generic) shape = SHAPE_GENERIC;   // run every statement through the term-table kernel (for cross-checks)
    ctx->shape = shape;
    ctx->D = D; ctx->points = points; ctx->ntables = ntables; ctx->nt_used = nt_used > 0 ? nt_used : 1;
    memset(&ctx->st, 0, sizeof ctx->st);
    ctx->st.nterms = nterms;
    int e = 0;
    for (int t = 0; t < nterms; t++) e = std::max(e, term_ptr[t + 1] - term_ptr[t] - 1);
    ctx->st_e = e;
    ctx->st_re = to_mont(pow_r(e));
    ctx->use_factor = false;
    for (int t = 0; t < nterms; t++) {
        // the GKR kernel reads lam from term 0
        const int at = shape == SHAPE_GKR ? (t == lam_term ? 0 : (t < lam_term ? t + 1 : t)) : (shape >= SHAPE_LISTED ? term_at[t] : t);
        DevTerm &tm = ctx->st.terms[at];
        tm.nf = (uint8_t)(term_ptr[t + 1] - term_ptr[t]);
        for (int k = 0; k < tm.nf; k++) tm.f[k] = (uint8_t)pos_of[term_tables[term_ptr[t] + k]];
        // c R^(m-1-e) for a term of m tables, c R^-e for the constant term
        const u32 scale = pow_r((tm.nf ? tm.nf - 1 : 0) - e);
        bool upper = false;
        u32 c[8];
        for (int k = 0; k < D; k++) {
            c[k] = (u32)(((u64)(coeffs[(size_t)t * D + k] % P) * scale) % P);
            if (k && c[k]) upper = true;
        }
        if (shape == SHAPE_GKR && !is_one(a_term)) {
            // a common coefficient ca in front: terms a and b become 1, lam becomes c_lam / ca, ca waits for the final factor
            if (t == lam_term) {
                u32 ca[8], inv[8], cl[8];
                for (int k = 0; k < D; k++) { ca[k] = to_mont(coeffs[(size_t)a_term * D + k] % P); cl[k] = c[k]; }
                ext_inv_host(D, ca, inv);
                ext_mul_host(D, cl, inv, c);   // canonical * Montgomery -> canonical
                upper = false;
                for (int k = 1; k < D; k++) upper = upper || c[k];
            } else {
                for (int k = 0; k < D; k++) { ctx->st_factor[k] = c[k]; c[k] = k == 0 ? 1u : 0u; }
                ctx->use_factor = true;
                upper = false;
            }
        }
        tm.ckind = upper ? CK_EXT : (c[0] == 1 ? CK_ONE : CK_BASE);
        for (int k = 0; k < D; k++) tm.coeff[k] = tm.nf ? to_mont(c[k]) : c[k];
        if (shape == SHAPE_PRODUCT) {   // the coefficient waits for the final factor
            ctx->use_factor = tm.ckind != CK_ONE;
            for (int k = 0; k < D; k++) ctx->st_factor[k] = c[k];
        }
    }
    // the kernel for rounds whose tables are all in the base field: terms with base coefficients share
    // one sum, a term with an extension coefficient has its own (at most one of those)
    {
        int ext_terms = 0, base_terms = 0;
        bool ok = true;
        for (int t = 0; t < nterms; t++) {
            DevTerm &tm = ctx->st.terms[t];
            if (tm.ckind == CK_EXT && tm.nf > 0) ext_terms++;
            else if (tm.ckind == CK_EXT) ok = false;          // an extension constant term
            else base_terms++;
        }
        if (ext_terms > 1 || nterms == 0 || nterms > BASE_MAX_TERMS || nt_used > 4 || points > FAST_POINTS) ok = false;
        for (int t = 0; t < nterms; t++) if (ctx->st.terms[t].nf > BASE_MAX_FACTORS) ok = false;
        ctx->base_groups = ok ? (base_terms > 0) + ext_terms : 0;
        memset(ctx->gcoef, 0, sizeof ctx->gcoef);
        ctx->gcoef[0][0] = R1;
        if (shape == SHAPE_PRODUCT) { ctx->base_groups = 1; ok = false; }   // the product's coefficient rides in the final factor
        if (shape >= SHAPE_LISTED) {   // a listed statement keeps the sums its entry says, whatever kind its coefficients happen to be
            ok = false;
            ctx->base_groups = listed_base_groups(shape);
            for (int e = 0; e < nterms && ctx->base_groups; e++)   // the terms lie in the entry's order by now
                if (listed_match->ck[e] == CK_EXT)
                    for (int c = 0; c < D; c++) ctx->gcoef[listed_base_group_of(shape, e)][c] = ctx->st.terms[e].coeff[c];
        }
        for (int t = 0; t < nterms && ok; t++) {
            DevTerm &tm = ctx->st.terms[t];
            tm.group = 0;
            if (tm.ckind == CK_EXT && tm.nf > 0) {
                tm.group = base_terms > 0 ? 1 : 0;
                for (int c = 0; c < D; c++) ctx->gcoef[tm.group][c] = tm.coeff[c];
            }
        }
    }
    {   // the small-value rounds: what the base-table kernel takes (its groups and descriptors), up to three tables and degree three
        bool ok = nterms >= 1 && nterms <= BASE_MAX_TERMS && nt_used >= 1 && nt_used <= 3 && points <= 3 && ctx->base_groups > 0;
        for (int t = 0; t < nterms && ok; t++) ok = ctx->st.terms[t].nf <= BASE_MAX_FACTORS;
        if (shape == SHAPE_PRODUCT) ok = nt_used <= 3;   // its coefficient, whatever it is, rides in the final factor
        ctx->sv_statement = ok;
    }
    ctx->have_statement = true;
    ctx->begun = false;
    return SC_OK;
}

// ------------------------------------------------------------------ tables

static int table_slot(sc_ctx *ctx, int slot, uint64_t entries, int stride) {
    if (!ctx) return SC_EINVAL;
    if (slot < 0 || slot >= SC_MAX_TABLES) return fail(ctx, SC_EINVAL, "table slot %d: expected 0..%d", slot, SC_MAX_TABLES - 1);
    if (stride != 1 && stride != 4 && stride != 8) return fail(ctx, SC_EINVAL, "stride %d: expected 1 or the extension degree", stride);
    if (entries == 0) return fail(ctx, SC_EINVAL, "empty table");
    cudaSetDevice(ctx->device);
    tail_stop(ctx);
    TableState &t = ctx->tab[slot];
    if (t.borrowed) { t.t0 = nullptr; t.t0_cap = 0; t.borrowed = false; }
    int rc = ensure(ctx, &t.t0, &t.t0_cap, entries * (u64)stride * 4);
    if (rc) return rc;
    t.entries = entries; t.stride = stride;
    ctx->begun = false;
    return SC_OK;
}

extern "C" int sc_borrow_table(sc_ctx *ctx, int slot, const uint32_t *table_dev, uint64_t entries, int stride) {
    if (!ctx) return SC_EINVAL;
    if (slot < 0 || slot >= SC_MAX_TABLES) return fail(ctx, SC_EINVAL, "table slot %d: expected 0..%d", slot, SC_MAX_TABLES - 1);
    if (stride != 1 && stride != 4 && stride != 8) return fail(ctx, SC_EINVAL, "stride %d: expected 1 or the extension degree", stride);
    if (!table_dev || entries == 0) return fail(ctx, SC_EINVAL, "empty table");
    if ((uintptr_t)table_dev % 16) return fail(ctx, SC_EINVAL, "a borrowed table must start on a 16-byte boundary");
    cudaSetDevice(ctx->device);
    tail_stop(ctx);
    TableState &t = ctx->tab[slot];
    if (!t.borrowed) dev_free(ctx, t.t0, t.t0_cap);
    t.t0 = const_cast<u32 *>(table_dev); t.t0_cap = 0; t.borrowed = true;
    t.entries = entries; t.stride = stride;
    ctx->begun = false;
    return SC_OK;
}

extern "C" int sc_upload_table(sc_ctx *ctx, int slot, const uint32_t *host, uint64_t entries, int stride) {
    if (!host) return SC_EINVAL;
    int rc = table_slot(ctx, slot, entries, stride);
    if (rc) return rc;
    TableState &t = ctx->tab[slot];
    CU(cudaMemcpyAsync(t.t0, host, entries * (u64)stride * 4, cudaMemcpyHostToDevice, ctx->stream));
    CU(launch_reduce_words(t.t0, entries * (u64)stride, ctx->stream));   // COERCE-EXT reduces its input
    ctx->launches++;
    // from pinned memory the copy reads the caller's buffer until it is done; from pageable memory the copy call
    // returns once the data has left it, and the rest is ordered on the stream
    cudaPointerAttributes at;
    const bool pageable = cudaPointerGetAttributes(&at, host) != cudaSuccess || at.type == cudaMemoryTypeUnregistered;
    cudaGetLastError();
    if (!pageable) CU(cudaStreamSynchronize(ctx->stream));
    return SC_OK;
}

extern "C" int sc_generate_table(sc_ctx *ctx, int slot, uint64_t seed, int table_id, uint64_t first, uint64_t entries, int stride,
                                 int nonzero) {
    int rc = table_slot(ctx, slot, entries, stride);
    if (rc) return rc;
    CU(launch_generate(ctx->tab[slot].t0, seed, table_id, first, entries, stride, nonzero, ctx->stream));
    ctx->launches++;
    CU(cudaStreamSynchronize(ctx->stream));
    return SC_OK;
}

extern "C" int sc_fetch_table(sc_ctx *ctx, int slot, uint32_t *host, uint64_t words) {
    if (!ctx || !host || slot < 0 || slot >= SC_MAX_TABLES) return SC_EINVAL;
    TableState &t = ctx->tab[slot];
    if (!t.t0 || words > t.entries * (u64)t.stride) return fail(ctx, SC_EINVAL, "table %d holds %llu words", slot, (unsigned long long)(t.entries * (u64)t.stride));
    cudaSetDevice(ctx->device);
    CU(cudaMemcpyAsync(host, t.t0, words * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CU(cudaStreamSynchronize(ctx->stream));
    return SC_OK;
}

static int export_tables(sc_ctx *ctx, const int *slots, int count, u64 entries, u32 *host) {
    const int D = ctx->D;
    const u64 words = (u64)count * entries * D;
    if (!words) return SC_OK;
    if (ctx->export_cap < words * 4) {
        if (ctx->h_export) cudaFreeHost(ctx->h_export);
        ctx->h_export = nullptr;
        u64 cap = ctx->export_cap;
        int rc = ensure(ctx, &ctx->d_export, &cap, words * 4);
        ctx->export_cap = cap;
        if (rc) return rc;
        CU(cudaHostAlloc(&ctx->h_export, words * 4, cudaHostAllocDefault));
    }
    ExportArgs a;
    memset(&a, 0, sizeof a);
    a.ntables = count; a.count = entries; a.out = ctx->d_export;
    for (int k = 0; k < count; k++) {
        const TableState &t = ctx->tab[slots[k]];
        a.src[k] = t.cur; a.src_base[k] = t.cur_base;
    }
    CU(launch_export(D, a, ctx->stream));
    ctx->launches++;
    CU(cudaMemcpyAsync(ctx->h_export, ctx->d_export, words * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CU(cudaStreamSynchronize(ctx->stream));
    memcpy(host, ctx->h_export, words * 4);
    return SC_OK;
}

extern "C" int sc_download_table(sc_ctx *ctx, int slot, uint32_t *host, uint64_t cap, uint64_t *entries) {
    if (!ctx || slot < 0 || slot >= SC_MAX_TABLES || !ctx->D) return SC_EINVAL;
    TableState &t = ctx->tab[slot];
    if (!t.t0) return fail(ctx, SC_ESTATE, "table %d was never uploaded", slot);
    if (ctx->tail_active || ctx->chain_active) return fail(ctx, SC_ESTATE, "the rounds are running on the device: the folded tables are not available");
    if (ctx->begun && ctx->sv_ok && ctx->j >= 1 && ctx->j <= ctx->sv_l0)
        return fail(ctx, SC_ESTATE, "the first %d rounds ran from one pass over the tables: nothing is folded before round %d", ctx->sv_l0, ctx->sv_l0);
    cudaSetDevice(ctx->device);
    if (!ctx->begun) { t.cur = t.t0; t.cur_base = t.stride == 1; t.cur_entries = t.entries; t.cur_buf = -1; }
    if (entries) *entries = t.cur_entries;
    const u64 count = t.cur_entries < cap ? t.cur_entries : cap;
    if (!host || !count) return SC_OK;
    return export_tables(ctx, &slot, 1, count, host);
}

// ------------------------------------------------------------------ begin: the weights of every round

static int low_bits_cap(int D) { return D == 4 ? 11 : 10; }   // 2^a multipliers of 2 D words in shared memory: 64 KiB

// The split of the v = (variables after the round's own) eq variables of a round: the lower a of
// them index the low multipliers held in shared memory, the others the high weights.  Any split
// gives the same sums (SPLIT-WEIGHTS, src/sumcheck.lisp:43-49, splits in the middle).
static int split_bits(int D, int v) {
    if (v < 20) return 0;
    int a = v - 12;
    return a < low_bits_cap(D) ? a : low_bits_cap(D);
}

// The host transcript of the proof that follows (or NULL): with it the resident kernel of the last rounds
// copies the transcript's hash state when it starts and derives every challenge itself instead of waiting
// for the host; the caller goes on sending the sums and drawing the challenges as before, and sc_challenge
// checks that they are the device's.  The transcript must not be used for anything else between those calls.
extern "C" int sc_attach_transcript(sc_ctx *ctx, const sc_transcript *tr) {
    if (!ctx) return SC_EINVAL;
    ctx->attached = tr;
    return SC_OK;
}
// The same for a caller whose transcript is not an sc_transcript (a Lisp one): the hash state as it stands when the
// next sc_round is called.  It is used by that call, if it starts a chain, and forgotten either way.
extern "C" int sc_attach_transcript_state(sc_ctx *ctx, const uint32_t cv[8], const uint32_t pending[16], int fill, uint64_t blocks) {
    if (!ctx || !cv || !pending || fill < 0 || fill > 64) return SC_EINVAL;
    memset(ctx->state0, 0, sizeof ctx->state0);
    memcpy(ctx->state0, cv, 32);
    memcpy(ctx->state0 + 8, pending, 64);
    for (int b = fill; b < 64; b++) reinterpret_cast<unsigned char *>(ctx->state0 + 8)[b] = 0;
    ctx->state0[24] = (u32)fill; ctx->state0[25] = (u32)blocks; ctx->state0[26] = (u32)(blocks >> 32);
    ctx->have_state = true;
    return SC_OK;
}
extern "C" int sc_set_device_transcript(sc_ctx *ctx, int on) {
    if (!ctx) return SC_EINVAL;
    tail_stop(ctx);
    ctx->device_transcript = on != 0;
    return SC_OK;
}
// The transcript's hash state of this moment, for a chain that starts now; false without a transcript of the proof's degree.
static bool transcript_state_now(sc_ctx *ctx, u32 *state) {
    if (ctx->attached) {
        uint32_t cv[8], pending[16];
        int fill = 0;
        uint64_t blocks = 0;
        if (sc_transcript_state(ctx->attached, cv, pending, &fill, &blocks) != SC_OK || sc_transcript_degree(ctx->attached) != ctx->D) return false;
        memset(state, 0, B3_STATE_WORDS * 4);
        memcpy(state, cv, sizeof cv); memcpy(state + 8, pending, sizeof pending);
        state[24] = (u32)fill; state[25] = (u32)blocks; state[26] = (u32)(blocks >> 32);
        return true;
    }
    if (ctx->have_state) { memcpy(state, ctx->state0, B3_STATE_WORDS * 4); return true; }
    return false;
}

// Child INDEX of the context: a context of its own on the same device, made on first use and destroyed
// with its parent (the parts of a statement wider than one kernel run on them).
extern "C" int sc_child(sc_ctx *ctx, int index, sc_ctx **out) {
    if (!ctx || !out || index < 0 || index >= 64) return SC_EINVAL;
    while ((int)ctx->children.size() <= index) {
        sc_ctx *c = nullptr;
        int rc = sc_create(ctx->device, &c);
        if (rc) return fail(ctx, rc, "sc_child: cannot make context %d", (int)ctx->children.size());
        ctx->children.push_back(c);
    }
    *out = ctx->children[index];
    return SC_OK;
}

// Device memory of the context's own for a caller's scratch: grow-only, freed with the context, counted in
// the memory budget.  The contents survive until the next call that asks for more.
extern "C" int sc_workspace(sc_ctx *ctx, uint64_t bytes, void **out) {
    if (!ctx || !out) return SC_EINVAL;
    cudaSetDevice(ctx->device);
    int rc = ensure(ctx, &ctx->d_work, &ctx->work_cap, bytes);
    if (rc) return rc;
    *out = ctx->d_work;
    return SC_OK;
}

// Make room ahead of a run of proofs of growing size (the layers of a tree, smallest first): the folded
// tables' buffers and the weight tables for proofs of up to N variables over K blocks and NTABLES tables,
// so that no proof of the run has to free and allocate again.
extern "C" int sc_reserve(sc_ctx *ctx, int D, int n, int K, int ntables) {
    if (!ctx) return SC_EINVAL;
    if (D != 4 && D != 8) return fail(ctx, SC_EINVAL, "extension degree %d: expected 4 or 8", D);
    if (n < 0 || n > 40 || K < 1 || ntables < 1 || ntables > SC_MAX_TABLES) return fail(ctx, SC_EINVAL, "sc_reserve: n = %d, K = %d, %d tables", n, K, ntables);
    cudaSetDevice(ctx->device);
    tail_stop(ctx);
    const u64 entries = (u64)K << n;
    int rc;
    for (int s = 0; s < ntables; s++) {
        TableState &t = ctx->tab[s];
        if (t.cur_buf >= 0) { t.cur = nullptr; t.cur_buf = -1; ctx->begun = false; }   // a buffer in use may move
        if ((rc = ensure(ctx, &t.buf[0], &t.buf_cap[0], entries / 2 * D * 4))) return rc;
        if ((rc = ensure(ctx, &t.buf[1], &t.buf_cap[1], entries / 4 * D * 4))) return rc;
    }
    u64 words = 0;
    for (int j = 0; j < n; j++) {   // as sc_begin lays the weights out, with eq and block weights present
        const int v = n - 1 - j, a = split_bits(D, v);
        if (a > 0) words += ((u64)1 << a) * 2 * D;
        words += ((u64)1 << (v - a)) * (u64)K * D;
    }
    if ((rc = ensure(ctx, &ctx->d_weights, &ctx->weights_cap, (words ? words : 4) * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_chunks, &ctx->chunks_cap, (u64)(n > 0 ? n : 1) * 512 * D * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_eq, &ctx->eq_cap, (u64)(n > 0 ? n : 1) * D * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_bw, &ctx->bw_cap, (u64)K * D * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_descs, &ctx->descs_cap, (u64)(2 * n + 1) * sizeof(WeightDesc)))) return rc;
    return SC_OK;
}

extern "C" int sc_begin(sc_ctx *ctx, int n, const uint32_t *eq, int K, const uint32_t *block_weights) {
    if (!ctx) return SC_EINVAL;
    if (!ctx->have_statement) return fail(ctx, SC_ESTATE, "sc_begin before sc_set_statement");
    tail_stop(ctx);
    if (n < 0 || n > 40) return fail(ctx, SC_EINVAL, "n = %d", n);
    if (block_weights && K < 1) return fail(ctx, SC_EINVAL, "K = %d block weights", K);
    if (!block_weights) K = 1;
    static const bool trace = getenv("SABLE_B200_TRACE") != nullptr;   // the host time of each part on stderr
    const auto t_in = std::chrono::steady_clock::now();
    const int D = ctx->D, w = ctx->logw;
    if (ctx->world > 1 && n < w) return fail(ctx, SC_EUNSUPPORTED, "several GPUs: n >= log2(world)");
    cudaSetDevice(ctx->device);
    const int nloc = n - w;
    const u64 want = (u64)K << nloc;
    for (int s = 0; s < ctx->ntables; s++) {
        TableState &t = ctx->tab[s];
        if (!t.t0) return fail(ctx, SC_ESTATE, "table %d was never uploaded", s);
        if (t.entries != want) return fail(ctx, SC_EINVAL, "table %d has %llu entries: expected %llu", s, (unsigned long long)t.entries, (unsigned long long)want);
        if (t.stride != 1 && t.stride != D) return fail(ctx, SC_EINVAL, "table %d has stride %d: expected 1 or %d", s, t.stride, D);
        t.cur = t.t0; t.cur_buf = -1; t.cur_base = t.stride == 1; t.cur_entries = t.entries;
    }
    ctx->n = n; ctx->K = K; ctx->j = 0; ctx->nloc = nloc; ctx->have_r = false; ctx->have_eq = eq != nullptr;
    // gather once a slice is down to 2^GATHER_BITS entries: from there on a round is latency, and an
    // exchange per round would double it
    int GATHER_BITS = 13;
    if (const char *env = getenv("SABLE_B200_GATHER_BITS")) GATHER_BITS = std::max(0, std::min(30, atoi(env)));
    ctx->gather_round = ctx->world > 1 ? std::max(0, nloc - GATHER_BITS) : n;
    const int gather_round = ctx->gather_round;
    ctx->stats.clear();
    ctx->plan.assign(n, RoundPlan());

    // eq and block weights in Montgomery form
    // staged in the context, so that the copies below need no wait: the vectors live until the next sc_begin
    std::vector<u32> &eqm = ctx->stage_eq, &bwm = ctx->stage_bw;
    eqm.assign((size_t)(n > 0 ? n : 1) * D, 0); bwm.assign((size_t)K * D, 0);
    if (eq) for (size_t i = 0; i < (size_t)n * D; i++) eqm[i] = to_mont(eq[i] % P);
    if (block_weights) for (size_t i = 0; i < (size_t)K * D; i++) bwm[i] = to_mont(block_weights[i] % P);

    // the factor of this rank: eq(r[nloc .. n), rank)
    ctx->use_post = false;
    if (ctx->world > 1 && eq) {
        if (D == 4) {
            Ext<4> acc = eone_mont<4>(), one = eone_mont<4>();
            for (int k = 0; k < w; k++) {
                Ext<4> rk; for (int c = 0; c < 4; c++) rk.v[c] = eqm[(size_t)(nloc + k) * 4 + c];
                acc = emul<4>(acc, ((ctx->rank >> k) & 1) ? rk : esub<4>(one, rk));
            }
            for (int c = 0; c < 4; c++) ctx->post[c] = acc.v[c];
        } else {
            Ext<8> acc = eone_mont<8>(), one = eone_mont<8>();
            for (int k = 0; k < w; k++) {
                Ext<8> rk; for (int c = 0; c < 8; c++) rk.v[c] = eqm[(size_t)(nloc + k) * 8 + c];
                acc = emul<8>(acc, ((ctx->rank >> k) & 1) ? rk : esub<8>(one, rk));
            }
            for (int c = 0; c < 8; c++) ctx->post[c] = acc.v[c];
        }
        ctx->use_post = true;
    }

    // one LOW and one HIGH table per round
    std::vector<WeightDesc> &descs = ctx->stage_descs;
    descs.clear();
    u64 words = 0, total_entries = 0;
    // A statement over base tables may take its first rounds from one pass (below): that pass walks the weights of round 1
    // (or 2) with one thread per low weight, 256 to a thread block, and wants the thread blocks to divide the SMs evenly:
    // 2^10 low weights are four thread blocks' worth (148 = 4 x 37), 2^11 would leave four SMs idle.  Any split gives the same sums.
    bool pass_candidate = ctx->sv_statement && K == 1 && !ctx->force_generic;
    for (int s = 0; s < ctx->ntables && pass_candidate; s++) pass_candidate = ctx->tab[s].stride == 1;
    int pass_round = 1;   // the round whose weights the pass would walk: 2 where three rounds are likely (decided below)
    {
        const char *env = getenv("SABLE_B200_SMALL_VALUES");
        bool ext_term = false;
        for (int t = 0; t < ctx->st.nterms; t++) ext_term = ext_term || (ctx->st.terms[t].ckind == CK_EXT && ctx->st.terms[t].nf > 0);
        if (ctx->shape == SHAPE_PRODUCT) ext_term = false;
        const bool want3 = env && env[0] == '3' ? true : ctx->nt_used <= 2;
        if (want3 && !(env && env[0] == '2') && !ext_term && ctx->points <= 2 && ctx->shape != SHAPE_LISTED + 1) pass_round = 2;
    }
    for (int j = 0; j < n; j++) {
        RoundPlan &pl = ctx->plan[j];
        const bool local = j < gather_round;         // before the gather
        const int end = local ? nloc : n;            // eq variables of this stage end here
        const int v = end - 1 - j;
        const int blocks = K;                         // every block in every round: with several GPUs each rank holds its slice of each
        int a = split_bits(D, v);
        if (pass_candidate && j == pass_round && a > 10) a = 10;   // (the round after it, which binds the tables, is faster with 2^11)
        pl.logL = a;
        pl.use_low = eq && a > 0;
        const bool has_bw = block_weights != nullptr;
        pl.use_high = (eq && v - a > 0) || has_bw;   // a single high weight without block weights is 1
        if (pl.use_low) {
            WeightDesc d; d.out_word = words; d.entries = 1ull << a; d.start = j + 1; d.bits = a; d.kind = 1; d.blocks = 0;
            pl.low_word = words; words += d.entries * 2 * D; total_entries += d.entries; descs.push_back(d);
        }
        if (pl.use_high) {
            WeightDesc d; d.out_word = words; d.entries = 1ull << (v - a); d.start = j + 1 + a; d.bits = eq ? v - a : 0; d.kind = 0;
            d.blocks = has_bw ? blocks : 0;
            const u64 count = d.entries * (u64)(d.blocks ? d.blocks : 1);
            pl.high_word = words; words += count * D; total_entries += count; descs.push_back(d);
        }
    }
    int rc;
    const auto t_plan = std::chrono::steady_clock::now();
    if ((rc = ensure(ctx, &ctx->d_eq, &ctx->eq_cap, eqm.size() * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_bw, &ctx->bw_cap, bwm.size() * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_chunks, &ctx->chunks_cap, (u64)(n > 0 ? n : 1) * 512 * D * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_weights, &ctx->weights_cap, (words ? words : 4) * 4))) return rc;
    if ((rc = ensure(ctx, &ctx->d_descs, &ctx->descs_cap, (descs.size() ? descs.size() : 1) * sizeof(WeightDesc)))) return rc;
    CU(cudaMemcpyAsync(ctx->d_eq, eqm.data(), eqm.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    CU(cudaMemcpyAsync(ctx->d_bw, bwm.data(), bwm.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (!descs.empty()) CU(cudaMemcpyAsync(ctx->d_descs, descs.data(), descs.size() * sizeof(WeightDesc), cudaMemcpyHostToDevice, ctx->stream));
    const auto t_copied = std::chrono::steady_clock::now();
    if (eq && n > 0) { CU(launch_eq_chunks(D, ctx->d_eq, n, ctx->d_chunks, ctx->stream)); ctx->launches++; }
    if (total_entries) {
        CU(launch_weight_tables(D, ctx->d_chunks, ctx->d_descs, (int)descs.size(), ctx->d_bw, ctx->d_weights, total_entries, ctx->stream));
        ctx->launches++;
    }
    // rounds 0 and 1 from one pass, tables bound to both challenges on the way into round 2: a product of
    // base tables, large enough for split weights, on one GPU, one block
    {
        const char *env = getenv("SABLE_B200_SMALL_VALUES");
        // any statement over base tables whose coefficients are base-field elements: what the reference takes this way
        // (no constants, src/sumcheck.lisp:535-539), as far as the base-table kernel's descriptors reach
        bool ok = !(env && env[0] == '0') && !ctx->force_generic && ctx->sv_statement && K == 1 && n >= 3 && ctx->gather_round > 2 &&
                  small_values_supported(D, ctx->points + 1, ctx->nt_used) && ctx->plan[1].logL >= 8;
        for (int s = 0; s < ctx->ntables && ok; s++) ok = ctx->tab[s].stride == 1;
        ctx->sv_ok = ok;
        // three rounds from the pass where the grid stays small (degree at most two: 27 points) and every coefficient is a
        // base element, as the reference's choice goes (CHOOSE-SMALL-VALUE-KERNEL, src/sumcheck.lisp:450-455: the largest
        // L0 up to 3 whose kernel fits); SABLE_B200_SMALL_VALUES=2 keeps it at two
        bool ext_term = false;
        for (int t = 0; t < ctx->st.nterms; t++) ext_term = ext_term || (ctx->st.terms[t].ckind == CK_EXT && ctx->st.terms[t].nf > 0);
        if (ctx->shape == SHAPE_PRODUCT) ext_term = false;
        ctx->sv_l0 = 2;
        // (measured at n = 25-26, D = 4: three rounds against two are 1.54 / 1.66 ms for a product of two tables, 1.79 / 1.91 ms
        // for a listed statement over two, 1.77 / 1.77 ms for a term table over three: so three tables stay at two unless
        // SABLE_B200_SMALL_VALUES=3 asks)
        const bool want3 = env && env[0] == '3' ? true : ctx->nt_used <= 2;
        if (ok && want3 && !(env && env[0] == '2') && !ext_term && n >= 4 && ctx->gather_round > 3 && ctx->shape != SHAPE_LISTED + 1 &&
            small_values3_supported(D, ctx->points + 1, ctx->nt_used) && ctx->plan[2].logL >= 8)
            ctx->sv_l0 = 3;
        memset(ctx->sv_eq, 0, sizeof ctx->sv_eq);
        if (ok && eq) for (int v = 1; v < ctx->sv_l0; v++) for (int c = 0; c < D; c++) ctx->sv_eq[v][c] = eq[(size_t)v * D + c] % P;
    }
    ctx->begun = true;
    if (trace) {
        auto us = [](std::chrono::steady_clock::time_point a, std::chrono::steady_clock::time_point b) { return std::chrono::duration<double, std::micro>(b - a).count(); };
        const auto t_out = std::chrono::steady_clock::now();
        fprintf(stderr, "  sc_begin n = %d: plan %.1f us, copies %.1f us, weight kernels %.1f us\n", n, us(t_in, t_plan), us(t_plan, t_copied), us(t_copied, t_out));
    }
    return SC_OK;
}

// ------------------------------------------------------------------ rounds

static void challenge_words(const sc_ctx *ctx, u32 *out) {
    for (int c = 0; c < ctx->D; c++) out[c] = to_mont(ctx->r[c]);   // REDC(r R s) = r s
}

// Fold every table by the pending challenge with the stand-alone kernel (the last fold, and the
// fold before the gather).
static int fold_all(sc_ctx *ctx, const u32 *r_dev = nullptr) {
    const int D = ctx->D;
    FoldArgs a;
    memset(&a, 0, sizeof a);
    a.ntables = ctx->ntables;
    if (!a.ntables) return SC_OK;
    const TableState &t0 = ctx->tab[0];
    a.nout = t0.cur_entries / 2;
    if (r_dev) a.r_dev = r_dev; else challenge_words(ctx, a.r);
    for (int s = 0; s < ctx->ntables; s++) {
        TableState &t = ctx->tab[s];
        const int nb = t.cur_buf == 0 ? 1 : 0;
        int rc = ensure(ctx, &t.buf[nb], &t.buf_cap[nb], a.nout * D * 4);
        if (rc) return rc;
        a.src[s] = t.cur; a.src_base[s] = t.cur_base; a.dst[s] = t.buf[nb];
    }
    CU(launch_fold(D, a, ctx->stream));
    ctx->launches++;
    for (int s = 0; s < ctx->ntables; s++) {
        TableState &t = ctx->tab[s];
        const int nb = t.cur_buf == 0 ? 1 : 0;
        t.cur = t.buf[nb]; t.cur_buf = nb; t.cur_base = false; t.cur_entries = a.nout;
    }
    ctx->have_r = false;
    return SC_OK;
}

// Gather every rank's slice of each table into whole tables, alike on every rank (rank k holds
// entries [k N/W, (k+1) N/W) of each block, so a block's slices in rank order are the block: one all-gather per block).
static int gather_tables(sc_ctx *ctx) {
    const int D = ctx->D, K = ctx->K;
    for (int s = 0; s < ctx->ntables; s++) {
        TableState &t = ctx->tab[s];
        const u64 words = t.cur_entries * (u64)(t.cur_base ? 1 : D), slice = words / (u64)K;
        int rc = ensure(ctx, &ctx->d_gtab[s], &ctx->gtab_cap[s], (u64)ctx->world * words * 4);
        if (rc) return rc;
        for (int b = 0; b < K; b++) {
            ncclResult_t r = g_nccl.AllGather(t.cur + (u64)b * slice, ctx->d_gtab[s] + (u64)b * ctx->world * slice, (size_t)slice, NCCL_UINT32, ctx->comm, ctx->stream);
            if (r) return fail(ctx, SC_ECOMM, "ncclAllGather: %s", g_nccl.GetErrorString(r));
        }
        t.cur = ctx->d_gtab[s]; t.cur_buf = -1; t.cur_entries *= (u64)ctx->world;
    }
    return SC_OK;
}

// ---- host arithmetic on canonical extension elements (D = 4 or 8), for the handful of products the small-value rounds need
namespace {
struct EX { u32 v[8]; };
EX ex_mul(int D, const EX &a, const EX &b) {   // REDC(a * bR) = a b
    EX o = {};
    if (D == 4) {
        Ext<4> x, y;
        for (int c = 0; c < 4; c++) { x.v[c] = a.v[c]; y.v[c] = to_mont(b.v[c]); }
        const Ext<4> z = emul<4>(x, y);
        for (int c = 0; c < 4; c++) o.v[c] = z.v[c];
    } else {
        Ext<8> x, y;
        for (int c = 0; c < 8; c++) { x.v[c] = a.v[c]; y.v[c] = to_mont(b.v[c]); }
        const Ext<8> z = emul<8>(x, y);
        for (int c = 0; c < 8; c++) o.v[c] = z.v[c];
    }
    return o;
}
EX ex_add(const EX &a, const EX &b) { EX o; for (int c = 0; c < 8; c++) o.v[c] = fadd(a.v[c], b.v[c]); return o; }
EX ex_sub(const EX &a, const EX &b) { EX o; for (int c = 0; c < 8; c++) o.v[c] = fsub(a.v[c], b.v[c]); return o; }
EX ex_base(u32 x) { EX o = {{x, 0, 0, 0, 0, 0, 0, 0}}; return o; }
EX ex_scale(const EX &a, u32 s) { EX o; for (int c = 0; c < 8; c++) o.v[c] = (u32)(((u64)a.v[c] * s) % P); return o; }
EX ex_load(int D, const u32 *w) { EX o = {}; memcpy(o.v, w, 4 * (size_t)D); return o; }
u32 fp_inv(u32 a) { u64 r = 1, x = a; for (u64 e = P - 2; e; e >>= 1) { if (e & 1) r = r * x % P; x = x * x % P; } return (u32)r; }
}  // namespace

// Round J < L0 of the small-value rounds from the accumulators A and the challenges so far (SMALL-VALUE-SUMS,
// src/sumcheck.lisp:481-494): g_j(X) = sum_v sum_u L_v(rho) eq(r_(j+1..L0-1), u) A[v, X, u], v over {0..G-1}^j with the
// Lagrange basis on the nodes 0 .. d at rho_0 .. rho_(j-1) (LAGRANGE-TENSOR, :463-474), u over {0,1}^(L0-1-j).
static void sv_sums(sc_ctx *ctx, int j, uint32_t *sums) {
    const int D = ctx->D, G = ctx->points + 1, d = ctx->points, L0 = ctx->sv_l0;
    auto A = [&](int z) { return ex_load(D, ctx->sv_A + (size_t)z * D); };
    std::vector<EX> tensor{ex_base(1)};                 // index sum v_t G^t
    for (int t = 0; t < j; t++) {
        const EX rho = ex_load(D, ctx->sv_rho[t]);
        EX L[8];
        for (int v = 0; v <= d; v++) {
            EX num = ex_base(1);
            u32 den = 1;
            for (int k = 0; k <= d; k++) {
                if (k == v) continue;
                num = ex_mul(D, num, ex_sub(rho, ex_base((u32)k)));
                den = (u32)(((u64)den * (u32)((v - k + (long long)P) % P)) % P);
            }
            L[v] = ex_scale(num, fp_inv(den));
        }
        std::vector<EX> next(tensor.size() * (size_t)G);
        for (int v = 0; v < G; v++)
            for (size_t w = 0; w < tensor.size(); w++) next[w + tensor.size() * (size_t)v] = ex_mul(D, tensor[w], L[v]);
        tensor.swap(next);
    }
    std::vector<EX> eqs{ex_base(1)};                    // eq over the variables j+1 .. L0-1, bit t of u: variable j+1+t
    std::vector<int> radix{0};                          // the grid index of u: its bits as base-G digits
    for (int t = j + 1; t < L0; t++) {
        EX w1 = ex_base(1), w0 = ex_base(1);
        if (ctx->have_eq) { w1 = ex_load(D, ctx->sv_eq[t]); w0 = ex_sub(ex_base(1), w1); }
        const size_t count = eqs.size();
        int weight = 1;
        for (int k = j + 1; k < t; k++) weight *= G;
        eqs.resize(2 * count); radix.resize(2 * count);
        for (size_t u = 0; u < count; u++) {
            eqs[count + u] = ctx->have_eq ? ex_mul(D, eqs[u], w1) : eqs[u];
            radix[count + u] = radix[u] + weight;
            if (ctx->have_eq) eqs[u] = ex_mul(D, eqs[u], w0);
        }
    }
    int gj = 1;
    for (int t = 0; t < j; t++) gj *= G;
    for (int xi = 0; xi < ctx->points; xi++) {
        const int X = xi ? xi + 1 : 0;
        EX g = ex_base(0);
        for (size_t v = 0; v < tensor.size(); v++)
            for (size_t u = 0; u < eqs.size(); u++) {
                EX a = A((int)v + gj * X + gj * G * radix[u]);
                if (ctx->have_eq) a = ex_mul(D, a, eqs[u]);
                g = ex_add(g, j ? ex_mul(D, a, tensor[v]) : a);
            }
        memcpy(sums + (size_t)xi * D, g.v, 4 * (size_t)D);
    }
}

// Round 0 of the small-value rounds: the pass over the tables, then the round's sums from the accumulators.
static int sv_round0(sc_ctx *ctx, uint32_t *sums) {
    const int D = ctx->D, G = ctx->points + 1, L0 = ctx->sv_l0, Z = L0 == 3 ? G * G * G : G * G;
    const int flag_word = L0 == 3 ? SV3_FLAG : SV_FLAG;
    const RoundPlan &pl = ctx->plan[L0 - 1];   // the weights of round L0 - 1 cover the variables L0 .. n-1: those of the blocks
    SvArgs a;
    memset(&a, 0, sizeof a);
    u64 bytes = 0;
    for (int k = 0; k < ctx->nt_used; k++) { a.src[k] = ctx->tab[ctx->order[k]].t0; bytes += ctx->tab[ctx->order[k]].entries * 4; }
    a.nblocks = ctx->tab[ctx->order[0]].entries >> L0;
    a.logL = pl.logL; a.use_low = pl.use_low; a.use_high = pl.use_high;
    a.low = ctx->d_weights + pl.low_word; a.high = ctx->d_weights + pl.high_word;
    const bool sharded = ctx->world > 1;
    a.use_post = ctx->st_e > 0 || ctx->use_factor || (sharded && ctx->use_post);
    for (int c = 0; c < D; c++) a.post[c] = ctx->use_factor ? mmul(to_mont(ctx->st_factor[c]), ctx->st_re) : (c == 0 ? ctx->st_re : 0u);
    if (sharded && ctx->use_post) ext_mul_host(D, a.post, ctx->post, a.post);   // this rank's eq weight
    a.partials = ctx->d_partials; a.counter = ctx->d_counter;
    a.st = ctx->st;
    {   // one sum per grid point while every coefficient is a base element (or rides in the final factor: a product); with a
        // term whose coefficient is not, two: that term's products apart, multiplied by the coefficient at the end
        bool ext_term = false;
        for (int t = 0; t < ctx->st.nterms; t++) ext_term = ext_term || (ctx->st.terms[t].ckind == CK_EXT && ctx->st.terms[t].nf > 0);
        if (ctx->shape == SHAPE_PRODUCT) ext_term = false;
        a.ngroups = ext_term ? 2 : 1;
        a.use_gcoef = ext_term ? 1 : 0;
        memcpy(a.gcoef, ctx->gcoef, sizeof a.gcoef);
        if (ext_term && ctx->base_groups == 1) {   // no term with a base coefficient beside it: its sum is the second all the same
            memcpy(a.gcoef[1], ctx->gcoef[0], sizeof a.gcoef[1]);
            memset(a.gcoef[0], 0, sizeof a.gcoef[0]);
            a.gcoef[0][0] = R1;
            for (int t = 0; t < a.st.nterms; t++) if (a.st.terms[t].ckind == CK_EXT) a.st.terms[t].group = 1;
        }
    }
    a.seq = ++ctx->seq;
    if (sharded) {
        int rc;
        if (!ctx->d_sv && (rc = dev_alloc(ctx, (void **)&ctx->d_sv, SV3_MAX_WORDS * 4))) return rc;
        if (!ctx->d_gather && (rc = dev_alloc(ctx, (void **)&ctx->d_gather, (u64)ctx->world * SV3_MAX_WORDS * 4))) return rc;
        a.out_dev = ctx->d_sv;
    } else {
        a.out_host = ctx->h_sv_dev;
    }
    const u32 lchunks = (1u << a.logL) / ROUND_THREADS;
    const u64 NH = a.nblocks >> a.logL;
    u64 nhg = std::max<u64>(1, (u64)small_values_grid_x(D, G, a.ngroups, L0, ctx->sms) / lchunks);   // one wave of thread blocks
    if (nhg > NH) nhg = NH;
    const int grid = (int)(lchunks * nhg);
    if (ctx->timing) {
        while (ctx->ev.size() < 2) { cudaEvent_t e; CU(cudaEventCreate(&e)); ctx->ev.push_back(e); }
        CU(cudaEventRecord(ctx->ev[0], ctx->stream));
    }
    if (L0 == 3) CU(launch_small_values3(D, ctx->shape, G, ctx->nt_used, a, grid, ctx->stream));
    else CU(launch_small_values(D, ctx->shape, G, ctx->nt_used, a, grid, ctx->stream));
    ctx->launches++;
    if (ctx->timing) CU(cudaEventRecord(ctx->ev[1], ctx->stream));
    if (sharded) {   // every rank's accumulators, then their sum mod p
        ncclResult_t r = g_nccl.AllGather(ctx->d_sv, ctx->d_gather, (size_t)Z * D, NCCL_UINT32, ctx->comm, ctx->stream);
        if (r) return fail(ctx, SC_ECOMM, "ncclAllGather: %s", g_nccl.GetErrorString(r));
        CU(launch_sum_ranks(ctx->d_gather, ctx->world, Z * D, ctx->d_sv, ctx->h_sv_dev, flag_word, a.seq, ctx->stream));
        ctx->launches++;
    }
    if (!wait_word(ctx, ctx->h_sv + flag_word, a.seq)) {
        const bool aborted = sharded && !ctx->comm;
        CU(cudaStreamSynchronize(ctx->stream));
        return fail(ctx, aborted ? SC_ECOMM : SC_ECUDA, aborted ? "the exchange between the GPUs did not finish; the communicator was aborted" : "the small-value pass did not finish");
    }
    if (ctx->timing) {
        CU(cudaStreamSynchronize(ctx->stream));
        sc_round_stat st; CU(cudaEventElapsedTime(&st.kernel_ms, ctx->ev[0], ctx->ev[1]));
        st.bytes = bytes; st.pairs = a.nblocks * 2;
        ctx->stats.push_back(st);
    }
    memcpy(ctx->sv_A, ctx->h_sv, (size_t)Z * D * 4);
    sv_sums(ctx, 0, sums);
    ctx->have_r = false;
    ctx->j = 1;
    return SC_OK;
}

// Rounds 1 .. L0 - 1: the challenge of the round before joins the others, the sums come from the accumulators.
static int sv_round_next(sc_ctx *ctx, uint32_t *sums) {
    const int j = ctx->j;
    memcpy(ctx->sv_rho[j - 1], ctx->r, 4 * (size_t)ctx->D);
    sv_sums(ctx, j, sums);
    if (ctx->timing) { sc_round_stat st; st.kernel_ms = 0; st.bytes = 0; st.pairs = 0; ctx->stats.push_back(st); }
    ctx->have_r = false;
    ctx->j = j + 1;
    return SC_OK;
}

// The last rounds run in one resident launch when the tables (all their blocks together) are small and
// nobody asked for per-round timing.  J: the round that would be its first.
static bool tail_wanted(const sc_ctx *ctx, int j) {
    if (ctx->tail_bits <= 0 || ctx->timing || ctx->ntables < 1 || ctx->nt_used > 4 || ctx->points > FAST_POINTS) return false;
    if (ctx->ntables * ctx->K > ROUND_THREADS || ctx->ntables * ctx->K * ctx->D > TAIL_FINAL_WORDS) return false;   // one thread and D words per final entry
    if (ctx->n - j > TAIL_MAX_ROUNDS) return false;
    return ctx->tab[ctx->order[0]].cur_entries <= (1ull << ctx->tail_bits);
}

// Launch the resident kernel for the rounds J .. n-1.  FOLD: round J folds by the pending challenge first (else it reads
// the tables as they are: round 0, or the round after a gather).  CHAIN: it carries the transcript on itself, from STATE0
// (the host transcript's state, when it is the chain's first launch) or from the state the launch before it left.
static int tail_start(sc_ctx *ctx, int j, bool fold, bool chain, bool chain_first, const u32 *state0) {
    const int D = ctx->D;
    TailArgs a;
    memset(&a, 0, sizeof a);
    a.ntables = ctx->ntables;
    a.nrounds = ctx->n - j;
    a.blocks = ctx->K;
    a.nofold = fold ? 0 : 1;
    u64 entries = 0;
    for (int k = 0; k < ctx->ntables; k++) {
        TableState &t = ctx->tab[ctx->order[k]];
        entries = t.cur_entries;
        a.src[k] = t.cur; a.src_base[k] = t.cur_base;
        // the folded tables alternate between the two buffers, starting with the one the source is not in
        const int first = t.cur_buf == 0 ? 1 : 0;
        for (int b = 0; b < 2; b++) { int rc = ensure(ctx, &t.buf[b], &t.buf_cap[b], std::max<u64>(entries / 2, 1) * D * 4); if (rc) return rc; }
        if (t.cur_buf >= 0 && t.buf_cap[t.cur_buf] == 0) return fail(ctx, SC_ESTATE, "table buffer lost");
        a.src[k] = t.cur_buf >= 0 ? t.buf[t.cur_buf] : t.cur;
        a.buf[0][k] = t.buf[first]; a.buf[1][k] = t.buf[first ^ 1];
        ctx->tail_buf0[ctx->order[k]] = first;
    }
    ctx->tail_entries = entries;
    for (int k = 0; k < a.nrounds; k++) {
        const RoundPlan &pl = ctx->plan[j + k];
        if (pl.logL != 0 || pl.use_low) return fail(ctx, SC_ESTATE, "a split round in the tail");
        a.rd[k].npairs = fold ? entries >> (k + 2) : entries >> (k + 1);   // pairs summed: of the folded table, or (first round, no fold) of the table itself
        a.rd[k].high_word = pl.high_word;
        a.rd[k].use_high = pl.use_high;
    }
    if (!fold) {}   // no challenge yet
    else if (chain && !chain_first) a.r_dev = ctx->d_chal + (size_t)(j - 1) * 16;
    else challenge_words(ctx, a.r);
    a.weights = ctx->d_weights;
    a.st = ctx->st;
    a.use_post = ctx->st_e > 0 || ctx->use_factor;
    for (int c = 0; c < D; c++) a.post[c] = ctx->use_factor ? mmul(to_mont(ctx->st_factor[c]), ctx->st_re) : (c == 0 ? ctx->st_re : 0u);
    ctx->tail_seq = ctx->seq + 1;
    ctx->seq += TAIL_MAX_ROUNDS + 2;
    a.seq = ctx->tail_seq;
    a.host = ctx->h_tail_dev;
    a.poll_limit = ctx->tail_polls;
    ctx->tail_own = chain;
    if (chain) {
        a.own_transcript = 1;
        if (chain_first) memcpy(a.tstate0, state0, sizeof a.tstate0);
        else a.tstate = ctx->d_tstate;
    }
    // the words that carry their own mark once written: cleared here (the launch before is through with them: its
    // final entries were seen, or it was stopped and the stream drained)
    for (int k = 0; k < a.nrounds; k++) {
        volatile u32 *slot = ctx->h_tail + (size_t)k * TAIL_SLOT_WORDS;
        for (int c = 0; c < 32; c++) slot[c] = 0;
        for (int c = 0; c < 8; c++) slot[40 + c] = 0;
    }
    for (int c = 0; c < ctx->ntables * ctx->K * D; c++) ((volatile u32 *)ctx->h_tail)[TAIL_FINALS + c] = 0;
    ((volatile u32 *)ctx->h_tail)[TAIL_STATUS] = 0;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    CU(launch_tail(D, ctx->shape, ctx->points, ctx->nt_used, a, ctx->stream));
    ctx->launches++;
    ctx->tail_active = true;
    ctx->tail_first = j;
    ctx->tail_rounds = a.nrounds;
    ctx->tail_nofold = a.nofold;
    return SC_OK;
}

// The resident kernel gave up waiting for the challenge of its round DONE - 1 (the host was too slow, or
// launches are serialised, as under a profiler): the tables are as that round's fold left them, so the
// proof goes on with one launch per round, and the context stops using the resident kernel.
static bool tail_recover(sc_ctx *ctx, int done) {
    if (ctx->h_tail[TAIL_STATUS] != 2 || done < 1) return false;
    const int folds = done - ctx->tail_nofold;   // folds the kernel finished: none yet after a first round that had no challenge
    for (int s = 0; s < ctx->ntables && folds > 0; s++) {
        TableState &t = ctx->tab[s];
        const int b = ctx->tail_buf0[s] ^ ((folds - 1) & 1);
        t.cur = t.buf[b]; t.cur_buf = b; t.cur_base = false; t.cur_entries = ctx->tail_entries >> folds;
    }
    ctx->tail_active = false;
    ctx->tail_bits = 0;
    return true;
}

// A round of the resident kernel: wait for its sums to be posted.
static int tail_round(sc_ctx *ctx, uint32_t *sums) {
    const int k = ctx->j - ctx->tail_first;
    const u32 *slot = ctx->h_tail + (size_t)k * TAIL_SLOT_WORDS;
    const int W = ctx->points * ctx->D;
    if (!(ctx->tail_own ? wait_word(ctx, slot + 32, ctx->tail_seq + (u32)k) : wait_here(ctx, slot, W))) {
        if (!ctx->tail_own && tail_recover(ctx, k)) return sc_round(ctx, sums);
        ctx->tail_active = false;
        ctx->chain_active = false;
        ctx->begun = false;
        return fail(ctx, SC_ESTATE, "the device stopped waiting for a challenge (status %u)", ctx->h_tail[TAIL_STATUS]);
    }
    for (int c = 0; c < W; c++) sums[c] = slot[c] & ~TAIL_HERE;
    ctx->have_r = false;
    ctx->j++;
    return SC_OK;
}

// What a launched round kernel leaves for the host to wait on and to account.
struct RoundLaunch {
    u32 seq = 0;
    u64 bytes = 0, npairs = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
};

// Launch the kernel of round J on the current tables (FOLD: folded by the previous challenge on the way in) and move
// the tables' state on to what the kernel leaves.  CHAIN: the round is part of a chain (see RoundArgs::tstate): it
// takes its challenge from device memory (unless it is the chain's first launch: then from the host, with STATE0 the
// host transcript's hash state), does the transcript's part itself and posts to its slot of the chain's buffer.
static int enqueue_round(sc_ctx *ctx, int j, bool fold, bool chain, bool chain_first, const u32 *state0, RoundLaunch *out) {
    const int D = ctx->D, W = ctx->points * D;
    const bool bind2 = ctx->sv_ok && j == ctx->sv_l0;   // the round after the small-value rounds reads the base tables and binds all their challenges on the way in
    const int bind_bits = bind2 ? ctx->sv_l0 : 1;
    const bool local = ctx->world > 1 && j < ctx->gather_round;
    const int shrink = 1 << bind_bits;   // entries in per entry out of the fold
    const RoundPlan &pl = ctx->plan[j];
    int rc;

    RoundArgs a;
    memset(&a, 0, sizeof a);
    a.ntables = ctx->ntables;
    u64 in_entries = 0, bytes = 0;
    for (int k = 0; k < ctx->ntables; k++) {
        TableState &t = ctx->tab[ctx->order[k]];
        a.src[k] = t.cur; a.src_base[k] = t.cur_base;
        if (k == 0) in_entries = t.cur_entries;
        else if (t.cur_entries != in_entries) return fail(ctx, SC_ESTATE, "tables in different states");
        bytes += t.cur_entries * (u64)(t.cur_base ? 1 : D) * 4;
        if (fold) {
            const int nb = t.cur_buf == 0 ? 1 : 0;
            if ((rc = ensure(ctx, &t.buf[nb], &t.buf_cap[nb], in_entries / shrink * D * 4))) return rc;
            a.dst[k] = t.buf[nb];
            bytes += in_entries / shrink * (u64)D * 4;
        }
    }
    // a statement over five or seven tables runs the kernel for six or eight: the spare position repeats position 0
    for (int k = ctx->ntables; k < SC_MAX_TABLES; k++) { a.src[k] = a.src[0]; a.dst[k] = a.dst[0]; a.src_base[k] = a.src_base[0]; }
    a.npairs = fold ? in_entries / (2 * shrink) : in_entries / 2;
    if (fold) {
        if (chain && !chain_first) a.r_dev = ctx->d_chal + (size_t)(j - 1) * 16;
        else challenge_words(ctx, a.r);
    }
    if (bind2) {   // eq(rho_0 .. rho_(L0-1), b): bit t of b pairs with rho_t (EQ-TABLE, src/field.lisp:354-363); the last challenge is the pending one
        std::vector<EX> w{ex_base(1)};
        for (int t = 0; t < bind_bits; t++) {
            const EX rt = ex_load(D, t + 1 < bind_bits ? ctx->sv_rho[t] : ctx->r);
            const size_t count = w.size();
            w.resize(2 * count);
            for (size_t b = 0; b < count; b++) { w[count + b] = ex_mul(D, w[b], rt); w[b] = ex_sub(w[b], w[count + b]); }
        }
        for (size_t b = 0; b < w.size(); b++)
            for (int c = 0; c < D; c++) {
                if (bind_bits == 2) a.bind[b][c] = to_mont(w[b].v[c]);
                else a.bind3[b][c] = to_mont(w[b].v[c]);
            }
    }
    a.logL = pl.logL;
    a.use_low = pl.use_low; a.use_high = pl.use_high;
    a.low = ctx->d_weights + pl.low_word;
    a.high = ctx->d_weights + pl.high_word;
    a.st = ctx->st;
    // the final factor: R^e of the statement, a product statement's coefficient, and this rank's eq
    // weight while the tables are sharded
    {
        const bool rankw = local && ctx->use_post;
        a.use_post = ctx->st_e > 0 || rankw || ctx->use_factor;
        const u32 re = ctx->st_re;
        for (int c = 0; c < D; c++) a.post[c] = ctx->use_factor ? mmul(to_mont(ctx->st_factor[c]), re) : (c == 0 ? re : 0u);
        if (rankw) ext_mul_host(D, a.post, ctx->post, a.post);
    }
    a.partials = ctx->d_partials; a.counter = ctx->d_counter;
    a.out_dev = ctx->d_out;
    if (chain) {   // the transcript kernel behind this launch posts to the host
        a.seq = ctx->chain_seq + (u32)j;
        a.out_host = nullptr;
        a.chained = 1;
        a.dead = chain_first ? nullptr : ctx->d_tstate + CHAIN_DEAD;
    } else {
        a.seq = ++ctx->seq;
        a.out_host = local ? nullptr : ctx->h_out_dev;
    }
    bool all_base = !fold && ctx->base_groups > 0 && !ctx->force_generic;
    for (int k = 0; k < ctx->nt_used && all_base; k++) all_base = a.src_base[k];
    // sharded rounds: the last block exchanges the sums with the other ranks itself (peer stores), unless the
    // ranks could not open each other's memory: then NCCL carries them
    const bool fused_exchange = local && ctx->p2p;
    if (fused_exchange) {
        for (int r = 0; r < ctx->world; r++) a.mail[r] = ctx->mail[r];
        a.world = ctx->world; a.rank = ctx->rank; a.xseq = ++ctx->xseq;
        a.mail_polls = ctx->mail_polls;
        if (!chain) a.out_host = ctx->h_out_dev;
    }
    TranscriptArgs ta;
    if (chain) {
        memset(&ta, 0, sizeof ta);
        ta.sums = ctx->d_out; ta.W = W; ta.D = D;
        ta.tstate = ctx->d_tstate;
        ta.chal_dev = ctx->d_chal + (size_t)j * 16;
        ta.tinit = chain_first;
        if (chain_first) memcpy(ta.tstate0, state0, sizeof ta.tstate0);
        ta.out_host = ctx->h_chain_dev + (size_t)j * CHAIN_SLOT_WORDS;
        ta.seq = a.seq;
    }
    if (chain && local && !fused_exchange) return fail(ctx, SC_ESTATE, "a chained round without peer access");

    const u64 chunk = (1ull << a.logL) > (u64)ROUND_THREADS ? (1ull << a.logL) : (u64)ROUND_THREADS;
    u64 chunks = (a.npairs + chunk - 1) / chunk;
    u64 max_grid = (u64)ctx->sms * ctx->blocks_per_sm;
    if (all_base && ctx->blocks_per_sm == 2) max_grid = (u64)ctx->sms * round_base_blocks_per_sm(D, ctx->shape, ctx->points, ctx->base_groups);
    int grid = (int)(chunks < max_grid ? chunks : max_grid);
    if (grid < 1) grid = 1;
    const size_t smem = a.use_low ? ((size_t)1 << a.logL) * 2 * D * 4 : 0;

    if (ctx->timing) {
        while (ctx->ev.size() < 2) { cudaEvent_t e; CU(cudaEventCreate(&e)); ctx->ev.push_back(e); }
        out->e0 = ctx->ev[0]; out->e1 = ctx->ev[1];
        CU(cudaEventRecord(out->e0, ctx->stream));
    }
    if (all_base) {
        a.ngroups = ctx->base_groups;
        memcpy(a.gcoef, ctx->gcoef, sizeof a.gcoef);
        CU(launch_round_base(D, ctx->shape, ctx->points, ctx->nt_used, a.ngroups, a, grid, smem, ctx->stream));
    } else {
        CU(launch_round(D, ctx->shape, ctx->points, ctx->nt_used, bind2 ? bind_bits : (fold ? 1 : 0), a, grid, smem, ctx->stream));
    }
    ctx->launches++;
    if (ctx->timing) CU(cudaEventRecord(out->e1, ctx->stream));
    if (chain) {   // the transcript's part of the round, behind it
        CU(launch_transcript_round(ta, ctx->stream));
        ctx->launches++;
    }
    if (local && !fused_exchange) {   // the whole job's sums: all-gather of the ranks' words, then their sum mod p
        if (!ctx->d_gather) { if ((rc = dev_alloc(ctx, (void **)&ctx->d_gather, (u64)ctx->world * SV_MAX_WORDS * 4))) return rc; }
        ncclResult_t r = g_nccl.AllGather(ctx->d_out, ctx->d_gather, (size_t)W, NCCL_UINT32, ctx->comm, ctx->stream);
        if (r) return fail(ctx, SC_ECOMM, "ncclAllGather: %s", g_nccl.GetErrorString(r));
        CU(launch_sum_ranks(ctx->d_gather, ctx->world, W, ctx->d_out, ctx->h_out_dev, MAX_PARTIAL_WORDS, a.seq, ctx->stream));
        ctx->launches++;
    }
    if (fold) {   // the tables the next launch reads (everything is ordered on the stream)
        for (int k = 0; k < ctx->ntables; k++) {
            TableState &t = ctx->tab[ctx->order[k]];
            const int nb = t.cur_buf == 0 ? 1 : 0;
            t.cur = t.buf[nb]; t.cur_buf = nb; t.cur_base = false; t.cur_entries = in_entries / shrink;
        }
    }
    out->seq = a.seq; out->bytes = bytes; out->npairs = a.npairs;
    return SC_OK;
}

// Wait for the launch number WANT at WORD (the kernel posts it after its sums).  The wait is bounded; a failed or
// unfinished exchange between the GPUs ends with the communicator aborted and SC_ECOMM.
static int await_round(sc_ctx *ctx, int j, const u32 *word, u32 want) {
    const bool had_comm = ctx->comm != nullptr;
    const bool seen = wait_word(ctx, word, want);
    if (!seen && had_comm && !ctx->comm) {
        cudaStreamSynchronize(ctx->stream);
        ctx->chain_active = false;
        return fail(ctx, SC_ECOMM, "round %d: the exchange between the GPUs did not finish in %d s; the communicator was aborted", j, ctx->comm_timeout_s);
    }
    if (seen && (*(volatile const u32 *)word & EXCHANGE_FAILED)) {
        CU(cudaStreamSynchronize(ctx->stream));
        tail_stop(ctx);
        comm_abort(ctx);
        return fail(ctx, SC_ECOMM, "round %d: another rank's sums never arrived; the communicator was aborted", j);
    }
    if (!seen || ctx->timing) CU(cudaStreamSynchronize(ctx->stream));
    if (!seen && (*(volatile const u32 *)word & ~EXCHANGE_FAILED) != want) return fail(ctx, SC_ECUDA, "round %d: the kernel did not post its sums", j);
    return SC_OK;
}

// The transcript on the device is asked for and possible: a transcript (or its state) is at hand, nobody wants
// per-round timing, and with several GPUs the ranks can exchange their sums inside the kernels.
static bool chain_wanted(const sc_ctx *ctx) {
    if (!ctx->device_transcript || ctx->timing || ctx->n > CHAIN_MAX_ROUNDS) return false;
    if (!ctx->attached && !ctx->have_state) return false;
    if (ctx->attached && sc_transcript_degree(ctx->attached) != ctx->D) return false;
    return ctx->world == 1 || ctx->p2p;
}

// Enqueue every remaining round at once, from round ctx->j on: round kernels whose last block carries the transcript
// on, then the resident kernel for the small rounds.  Nothing here waits for the device.
static int chain_start(sc_ctx *ctx) {
    u32 state[B3_STATE_WORDS];
    if (!transcript_state_now(ctx, state)) return fail(ctx, SC_ESTATE, "no transcript state for the device to start from");
    const auto t_begin = std::chrono::steady_clock::now();
    ctx->have_state = false;
    const int j0 = ctx->j;
    ctx->chain_first = j0;
    ctx->chain_seq = ctx->seq + 1;
    ctx->seq += CHAIN_MAX_ROUNDS + 2;
    bool fold = ctx->have_r, first = true;
    int j = j0, rc;
    for (; j < ctx->n; j++) {
        const u32 *r_dev = first ? nullptr : ctx->d_chal + (size_t)(j - 1) * 16;
        if (ctx->world > 1 && j == ctx->gather_round) {   // the slices are small: gather them, every rank goes on alike
            if (fold && (rc = fold_all(ctx, r_dev))) return rc;
            if ((rc = gather_tables(ctx))) return rc;
            if (fold) {   // the fold is done: the round itself reads the gathered tables as they are ...
                // ... which the round kernels cannot know, so the tables go one more step: round j folds nothing
                fold = false;
            }
        }
        const bool local = ctx->world > 1 && j < ctx->gather_round;
        if (!local && tail_wanted(ctx, j)) {
            if ((rc = tail_start(ctx, j, fold, true, first, state))) return rc;
            break;
        }
        RoundLaunch L;
        if ((rc = enqueue_round(ctx, j, fold, true, first, state, &L))) return rc;
        first = false;
        fold = true;
    }
    ctx->chain_end = j;
    ctx->chain_active = true;
    ctx->have_r = false;
    ctx->chain_t0 = std::chrono::steady_clock::now();
    if (getenv("SABLE_B200_TRACE")) fprintf(stderr, "  chain of rounds %d..%d enqueued in %.1f us (%d round kernels)\n", j0, ctx->n - 1, std::chrono::duration<double, std::micro>(ctx->chain_t0 - t_begin).count(), j - j0);
    return SC_OK;
}

// A round of a chain: wait for its slot.
static int chain_round(sc_ctx *ctx, uint32_t *sums) {
    const int j = ctx->j;
    if (j >= ctx->chain_end) return tail_round(ctx, sums);
    const u32 *slot = ctx->h_chain + (size_t)j * CHAIN_SLOT_WORDS;
    int rc = await_round(ctx, j, slot + MAX_PARTIAL_WORDS, ctx->chain_seq + (u32)j);
    if (rc) { ctx->chain_active = false; ctx->begun = false; return rc; }
    static const bool trace = getenv("SABLE_B200_TRACE") != nullptr;
    if (trace) fprintf(stderr, "  chained round %d seen %.1f us after the chain was enqueued\n", j, std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - ctx->chain_t0).count());
    memcpy(sums, slot, (size_t)ctx->points * ctx->D * 4);
    ctx->have_r = false;
    ctx->j = j + 1;
    return SC_OK;
}

extern "C" int sc_round(sc_ctx *ctx, uint32_t *sums) {
    if (!ctx || !sums) return SC_EINVAL;
    if (!ctx->begun) return fail(ctx, SC_ESTATE, "sc_round before sc_begin");
    if (ctx->j >= ctx->n) return fail(ctx, SC_ESTATE, "all %d rounds are done", ctx->n);
    if (ctx->j > 0 && !ctx->have_r) return fail(ctx, SC_ESTATE, "round %d needs the challenge of round %d", ctx->j, ctx->j - 1);
    static const bool trace = getenv("SABLE_B200_TRACE") != nullptr;
    const auto tr0 = std::chrono::steady_clock::now();
    cudaSetDevice(ctx->device);
    const int D = ctx->D, j = ctx->j, W = ctx->points * D;
    if (ctx->chain_active) return chain_round(ctx, sums);
    if (ctx->tail_active) return tail_round(ctx, sums);
    if (ctx->sv_ok && j == 0) return sv_round0(ctx, sums);
    if (ctx->sv_ok && j < ctx->sv_l0) return sv_round_next(ctx, sums);
    if (!round_supported(D, ctx->points, ctx->nt_used)) return fail(ctx, SC_EUNSUPPORTED, "no kernel for D=%d points=%d tables=%d", D, ctx->points, ctx->nt_used);
    int rc;
    if (chain_wanted(ctx)) {
        if ((rc = chain_start(ctx))) return rc;
        return chain_round(ctx, sums);
    }
    ctx->have_state = false;   // a state handed over for this call and not used
    bool fold = ctx->have_r;
    if (ctx->world > 1 && j == ctx->gather_round) {   // the slices are small: gather them, every rank goes on alike
        if (fold && (rc = fold_all(ctx))) return rc;
        if ((rc = gather_tables(ctx))) return rc;
        fold = false;   // folded already (fold_all cleared the pending challenge)
    }
    const bool local = ctx->world > 1 && j < ctx->gather_round;
    if (!local && tail_wanted(ctx, j)) {
        if ((rc = tail_start(ctx, j, fold, false, false, nullptr))) return rc;
        ctx->have_r = false;
        return tail_round(ctx, sums);
    }
    const auto tr1 = std::chrono::steady_clock::now();
    RoundLaunch L;
    if ((rc = enqueue_round(ctx, j, fold, false, false, nullptr, &L))) return rc;
    const auto tr2 = std::chrono::steady_clock::now();
    // wait for the sums: poll the word the kernel posts after them (a stream synchronize costs several
    // microseconds more per round); the wait is bounded
    if ((rc = await_round(ctx, j, ctx->h_out + MAX_PARTIAL_WORDS, L.seq))) return rc;
    memcpy(sums, ctx->h_out, (size_t)W * 4);
    if (trace) {
        const auto tr3 = std::chrono::steady_clock::now();
        auto us = [](std::chrono::steady_clock::time_point x, std::chrono::steady_clock::time_point y) { return std::chrono::duration<double, std::micro>(y - x).count(); };
        fprintf(stderr, "  sc_round %d: prepare %.1f us, launch %.1f us, wait %.1f us\n", j, us(tr0, tr1), us(tr1, tr2), us(tr2, tr3));
    }
    if (ctx->timing) {
        sc_round_stat s;
        CU(cudaEventElapsedTime(&s.kernel_ms, L.e0, L.e1));
        s.bytes = L.bytes; s.pairs = L.npairs;
        ctx->stats.push_back(s);
    }
    ctx->have_r = false;
    ctx->j = j + 1;
    return SC_OK;
}

extern "C" int sc_challenge(sc_ctx *ctx, const uint32_t *r) {
    if (!ctx || !r) return SC_EINVAL;
    if (!ctx->begun || ctx->j == 0) return fail(ctx, SC_ESTATE, "sc_challenge before the first round");
    if (ctx->have_r) return fail(ctx, SC_ESTATE, "round %d already has its challenge", ctx->j - 1);
    for (int c = 0; c < ctx->D; c++) ctx->r[c] = r[c] % P;
    ctx->have_r = true;
    const int done = ctx->j - 1;   // the round the challenge belongs to
    if (ctx->chain_active && done >= ctx->chain_first && done < ctx->chain_end) {
        // the round kernel derived this challenge itself and posted it with its sums: it must be the caller's
        const volatile u32 *slot = ctx->h_chain + (size_t)done * CHAIN_SLOT_WORDS;
        for (int c = 0; c < ctx->D; c++)
            if (slot[CHAIN_CHAL_WORD + c] != ctx->r[c]) {
                tail_stop(ctx);
                ctx->begun = false;
                return fail(ctx, SC_ESTATE, "round %d: the challenge differs from the one the device derived from the attached transcript (was the transcript used for something else during the proof?)", done);
            }
        return SC_OK;
    }
    if (ctx->tail_active && ctx->tail_own) {
        // the resident kernel derived this challenge itself from its copy of the transcript: it must be the caller's
        const u32 k = (u32)(done - ctx->tail_first);
        const u32 *slot = ctx->h_tail + (size_t)k * TAIL_SLOT_WORDS;
        if (!wait_word(ctx, slot + 50, ctx->tail_seq + k)) return fail(ctx, SC_ECUDA, "the device did not post its challenge of round %d", done);
        for (int c = 0; c < ctx->D; c++)
            if (((volatile const u32 *)slot)[52 + c] != ctx->r[c]) {
                tail_stop(ctx);
                ctx->begun = false;
                return fail(ctx, SC_ESTATE, "round %d: the challenge differs from the attached transcript's (was the transcript used for something else during the proof?)", done);
            }
        return SC_OK;
    }
    if (ctx->tail_active) {   // hand the challenge to the resident kernel: it polls the words themselves, each marked as written
        u32 *slot = ctx->h_tail + (size_t)(done - ctx->tail_first) * TAIL_SLOT_WORDS;
        for (int c = 0; c < ctx->D; c++) ((volatile u32 *)slot)[40 + c] = ctx->r[c] | TAIL_HERE;
        std::atomic_thread_fence(std::memory_order_seq_cst);
    }
    return SC_OK;
}

extern "C" int sc_finish(sc_ctx *ctx, uint32_t *folded) {
    if (!ctx) return SC_EINVAL;
    if (!ctx->begun) return fail(ctx, SC_ESTATE, "sc_finish before sc_begin");
    if (ctx->j != ctx->n) return fail(ctx, SC_ESTATE, "%d of %d rounds done", ctx->j, ctx->n);
    if (ctx->n > 0 && !ctx->have_r) return fail(ctx, SC_ESTATE, "the last round has no challenge");
    cudaSetDevice(ctx->device);
    int rc;
    if (ctx->tail_active) {   // the resident kernel folds by the last challenge and posts the final entries
        const auto t_in = std::chrono::steady_clock::now();
        const bool ok = wait_here(ctx, ctx->h_tail + TAIL_FINALS, ctx->ntables * ctx->K * ctx->D);
        // posting them was the launch's last act (its reads and writes of the tables are done, its status is written): no
        // need to wait for the stream to drain, whatever follows on it is ordered behind the launch anyway
        if (!ok) CU(cudaStreamSynchronize(ctx->stream));
        if (getenv("SABLE_B200_TRACE"))
            fprintf(stderr, "  sc_finish: final entries after %.1f us\n", std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_in).count());
        if (ok && ctx->tail_own && getenv("SABLE_B200_TRACE"))
            for (int k = 0; k < ctx->tail_rounds; k++) {
                const u32 *slot = ctx->h_tail + (size_t)k * TAIL_SLOT_WORDS;
                fprintf(stderr, "  resident round %d: arithmetic %u ns, transcript %u ns\n", ctx->tail_first + k, slot[60], slot[61]);
            }
        if (ok) {
            ctx->tail_active = false;
            ctx->chain_active = false;
            ctx->begun = false;
            if (folded) {
                const size_t KD = (size_t)ctx->K * ctx->D;   // per table: K entries
                for (int k = 0; k < ctx->ntables; k++)
                    for (size_t c = 0; c < KD; c++) folded[(size_t)ctx->order[k] * KD + c] = ctx->h_tail[TAIL_FINALS + (size_t)k * KD + c] & ~TAIL_HERE;
            }
            return SC_OK;
        }
        if (!tail_recover(ctx, ctx->tail_rounds)) {   // else: the last fold below, by the challenge it did not wait for
            ctx->tail_active = false;
            ctx->begun = false;
            return fail(ctx, SC_ESTATE, "the device stopped waiting for a challenge (status %u)", ctx->h_tail[TAIL_STATUS]);
        }
    }
    if (ctx->n > 0 && (rc = fold_all(ctx))) return rc;
    if (folded && ctx->ntables) {
        int slots[SC_MAX_TABLES];
        for (int s = 0; s < ctx->ntables; s++) slots[s] = s;
        if ((rc = export_tables(ctx, slots, ctx->ntables, (u64)ctx->K, folded))) return rc;
    }
    ctx->chain_active = false;
    ctx->begun = false;
    return SC_OK;
}

// ------------------------------------------------------------------ several GPUs

extern "C" int sc_comm_unique_id(void *nccl_id128) {
    if (!nccl_id128) return SC_EINVAL;
    if (!g_nccl.load()) return SC_ECOMM;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id)) return SC_ECOMM;
    memcpy(nccl_id128, &id, sizeof id);
    return SC_OK;
}

extern "C" int sc_comm_info(const sc_ctx *ctx, int *rank, int *world) {
    if (!ctx) return SC_EINVAL;
    if (rank) *rank = ctx->rank;
    if (world) *world = ctx->world;
    return SC_OK;
}

extern "C" int sc_comm_init(sc_ctx *ctx, const void *nccl_id128, int rank, int world) {
    if (!ctx || !nccl_id128) return SC_EINVAL;
    if (world < 1 || (world & (world - 1)) || rank < 0 || rank >= world) return fail(ctx, SC_EINVAL, "rank %d of %d: the world must be a power of two", rank, world);
    if (ctx->comm) return fail(ctx, SC_ESTATE, "the context already has a communicator");
    if (!g_nccl.load()) return fail(ctx, SC_ECOMM, "cannot load libnccl.so.2: %s", dlerror());
    cudaSetDevice(ctx->device);
    ncclUniqueId id;
    memcpy(&id, nccl_id128, sizeof id);
    ncclResult_t r = g_nccl.CommInitRank(&ctx->comm, world, id, rank);
    if (r) { ctx->comm = nullptr; return fail(ctx, SC_ECOMM, "ncclCommInitRank: %s", g_nccl.GetErrorString(r)); }
    ctx->rank = rank; ctx->world = world;
    ctx->logw = 0;
    while ((1 << ctx->logw) < world) ctx->logw++;
    ctx->begun = false;
    // mailboxes: every rank makes one, the handles go round with an all-gather, every rank opens the others'
    const char *env = getenv("SABLE_B200_P2P");
    if (world > 1 && world <= 8 && !(env && env[0] == '0')) {
        const size_t bytes = (size_t)2 * world * MAIL_WORDS * 4;
        u32 *own = nullptr, *d_handles = nullptr;
        cudaIpcMemHandle_t mine, all[8];
        bool ok = cudaMalloc(&own, bytes) == cudaSuccess && cudaMemset(own, 0, bytes) == cudaSuccess &&
                  cudaIpcGetMemHandle(&mine, own) == cudaSuccess &&
                  cudaMalloc(&d_handles, (size_t)(world + 1) * sizeof mine) == cudaSuccess &&
                  cudaMemcpy(d_handles + (size_t)world * (sizeof mine / 4), &mine, sizeof mine, cudaMemcpyHostToDevice) == cudaSuccess;
        if (ok) ok = g_nccl.AllGather(d_handles + (size_t)world * (sizeof mine / 4), d_handles, sizeof mine / 4, NCCL_UINT32, ctx->comm, ctx->stream) == 0 &&
                     cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
                     cudaMemcpy(all, d_handles, (size_t)world * sizeof mine, cudaMemcpyDeviceToHost) == cudaSuccess;
        for (int p = 0; p < world && ok; p++) {
            if (p == rank) { ctx->mail[p] = own; continue; }
            void *ptr = nullptr;
            ok = cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
            ctx->mail[p] = (u32 *)ptr;
        }
        if (d_handles) cudaFree(d_handles);
        if (!ok) {   // no peer access: the sums go through NCCL instead
            cudaGetLastError();
            for (int p = 0; p < world; p++) { if (ctx->mail[p] && p != rank) cudaIpcCloseMemHandle(ctx->mail[p]); ctx->mail[p] = nullptr; }
            if (own) cudaFree(own);
        }
        ctx->p2p = ok;
        ctx->xseq = 0;
    }
    return SC_OK;
}

// ------------------------------------------------------------------ a round without any allocation
//
// sc_round_sums_static is for callers that must not allocate device memory while they run: code
// between the capture calls of a stream, a service whose memory pool was sized up front and
// handed out completely, a plug-in that is given device pointers but no allocator.  A context
// (sc_create) allocates its partial-sum buffers and grows table buffers on demand; this entry
// point takes everything from the caller and keeps its only scratch -- one row of partial sums
// per block and the counter of finished blocks -- in the fixed array below, which every GPU that
// loads the library holds until the process ends.

namespace {
constexpr int STATIC_ROWS = 2048;                 // blocks a call may launch: one partial row each
constexpr u64 STATIC_PAIRS_PER_ROW = 65536;       // pairs a block sums
constexpr int STATIC_HEAD_WORDS = 64;             // the counter, in 256 bytes of its own
constexpr int STATIC_ROW_WORDS = 32;              // points * D words per row: degree <= 4 at D = 8, <= 8 at D = 4
constexpr int STATIC_WORDS = STATIC_HEAD_WORDS + STATIC_ROWS * STATIC_ROW_WORDS;   // 64 + 2048 * 32 words = 256.25 KiB
static __device__ __align__(256) u32 g_static_scratch[STATIC_WORDS];
constexpr int STATIC_MAX_DEVICES = 64;
std::atomic<u32 *> g_static_ptr[STATIC_MAX_DEVICES];   // the array's device address, per device ordinal (null = not asked yet)
std::atomic<int> g_static_sms[STATIC_MAX_DEVICES];     // the device's SM count, asked at the same time
}  // namespace

static int round_sums_static(sc_ctx *ctx, int D, int points, int ntables, const uint32_t *const *tables_dev, const int *strides,
                             uint64_t entries, int nterms, const uint32_t *coeffs, const int32_t *term_ptr,
                             const int32_t *term_tables, uint32_t *sums_dev, void *stream);

extern "C" int sc_round_sums_static(int D, int points, int ntables, const uint32_t *const *tables_dev, const int *strides,
                                    uint64_t entries, int nterms, const uint32_t *coeffs, const int32_t *term_ptr,
                                    const int32_t *term_tables, uint32_t *sums_dev, void *stream, char *message,
                                    size_t message_cap) {
    // the statement is lowered into a context of this call's own (it never owns device memory), so calls
    // from different host threads share nothing on the host but the table of scratch addresses below
    sc_ctx lowering;
    sc_ctx *ctx = &lowering;
    if (message && message_cap) message[0] = 0;
    const int rc = round_sums_static(ctx, D, points, ntables, tables_dev, strides, entries, nterms, coeffs, term_ptr, term_tables,
                                     sums_dev, stream);
    if (rc && message && message_cap) snprintf(message, message_cap, "%s", ctx->last_error.c_str());
    return rc;
}

static int round_sums_static(sc_ctx *ctx, int D, int points, int ntables, const uint32_t *const *tables_dev, const int *strides,
                             uint64_t entries, int nterms, const uint32_t *coeffs, const int32_t *term_ptr,
                             const int32_t *term_tables, uint32_t *sums_dev, void *stream) {
    if (!tables_dev || !strides || !sums_dev) return fail(ctx, SC_EINVAL, "null argument");
    if (entries < 2 || (entries & 1)) return fail(ctx, SC_EINVAL, "%llu entries: expected an even number", (unsigned long long)entries);
    const u64 npairs = entries / 2;
    const u64 rows = (npairs + STATIC_PAIRS_PER_ROW - 1) / STATIC_PAIRS_PER_ROW;
    if (rows > (u64)STATIC_ROWS)
        return fail(ctx, SC_EINVAL, "%llu entries need %llu rows of scratch: the static array holds %d (at most %llu entries per table)",
                    (unsigned long long)entries, (unsigned long long)rows, STATIC_ROWS,
                    (unsigned long long)(2 * STATIC_PAIRS_PER_ROW * STATIC_ROWS));
    if ((u64)points * (u64)D > (u64)STATIC_ROW_WORDS) return fail(ctx, SC_EUNSUPPORTED, "points * D = %d: the static rows hold %d words", points * D, STATIC_ROW_WORDS);
    int rc = sc_set_statement(ctx, D, points, ntables, nterms, coeffs, term_ptr, term_tables);
    if (rc) return rc;
    if (!round_supported(D, ctx->points, ctx->nt_used)) return fail(ctx, SC_EUNSUPPORTED, "no kernel for D=%d points=%d tables=%d", D, points, ctx->nt_used);
    for (int t = 0; t < ntables; t++) {
        if (!tables_dev[t] || (strides[t] != 1 && strides[t] != D)) return fail(ctx, SC_EINVAL, "table %d: null, or stride %d not 1 or %d", t, strides[t], D);
        // the kernel reads pairs of base entries as 8-byte words and extension entries as 16-byte words
        if ((uintptr_t)tables_dev[t] % 16) return fail(ctx, SC_EINVAL, "table %d does not start on a 16-byte boundary", t);
    }
    if ((uintptr_t)sums_dev % 4) return fail(ctx, SC_EINVAL, "the sums do not start on a 4-byte boundary");

    // set-up, once per device: the array's name is a host-side stand-in, the kernel needs its device address
    int device = -1;
    CU(cudaGetDevice(&device));
    if (device < 0 || device >= STATIC_MAX_DEVICES) return fail(ctx, SC_EUNSUPPORTED, "device ordinal %d", device);
    u32 *scratch = g_static_ptr[device].load(std::memory_order_acquire);
    int sms = g_static_sms[device].load(std::memory_order_acquire);
    if (!scratch) {   // two threads that both find it unset both ask, and store the same answer
        CU(cudaGetSymbolAddress((void **)&scratch, g_static_scratch));
        CU(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        g_static_sms[device].store(sms, std::memory_order_release);
        g_static_ptr[device].store(scratch, std::memory_order_release);
    }
    cudaStream_t s = (cudaStream_t)stream;
    // the array keeps what the last call left: the counter must start at zero
    CU(cudaMemsetAsync(scratch, 0, STATIC_HEAD_WORDS * 4, s));

    RoundArgs a;
    memset(&a, 0, sizeof a);
    a.ntables = ctx->nt_used;
    for (int k = 0; k < ctx->nt_used; k++) {
        a.src[k] = tables_dev[ctx->order[k]];
        a.src_base[k] = strides[ctx->order[k]] == 1;
    }
    // a statement over five or seven tables runs the kernel for six or eight: the spare position repeats position 0
    for (int k = ctx->nt_used; k < SC_MAX_TABLES; k++) { a.src[k] = a.src[0]; a.src_base[k] = a.src_base[0]; }
    a.npairs = npairs;
    a.st = ctx->st;
    a.use_post = ctx->st_e > 0 || ctx->use_factor;
    const u32 re = to_mont(pow_r(ctx->st_e));
    for (int c = 0; c < D; c++) a.post[c] = ctx->use_factor ? mmul(to_mont(ctx->st_factor[c]), re) : (c == 0 ? re : 0u);
    a.counter = scratch;
    a.partials = scratch + STATIC_HEAD_WORDS;
    a.out_dev = sums_dev;
    // blocks: one per chunk of 256 pairs up to two per SM, and never more than the array has rows
    const u64 chunks = (npairs + ROUND_THREADS - 1) / ROUND_THREADS;
    u64 grid = std::min<u64>(chunks, (u64)2 * (u64)(sms > 0 ? sms : 148));
    grid = std::max<u64>(1, std::min<u64>(grid, (u64)STATIC_ROWS));
    CU(launch_round(D, ctx->shape, ctx->points, ctx->nt_used, false, a, (int)grid, 0, s));
    return SC_OK;
}
