// N-sharded multi-GPU GEMM behind the C ABI, for ONE host process that drives all GPUs of a box
// (maize_mgpu_create / maize_gemm_bf16_nsharded / maize_gemm_bf16_nsharded_host / maize_mgpu_destroy,
// declared in include/maize_gemm.h).
//
// The reference has no multi-GPU code; a caller that binds where its GEMM entry point sits
// (crates/maize_tile/src/gemm/mod.rs:37-55) gets here the split of B's column panels
// (crates/maize_tile/src/gmem/col_panel.rs:88-124) lifted across GPUs: device g owns a contiguous block of rows
// of B (N x K, K-major) and produces the matching column block of C; A is replicated from a root device every
// call; there is no reduction and C stays sharded.
//
// Transport: the copy-engine chain.  The devices are chained from the root in index order; every device forwards
// A to the next one in row chunks with device-to-device copies into the next device's landing buffer (peer access,
// no SM touches the bytes) and counts the forwarded chunks in a flag word there; a device forwards a chunk as
// soon as its own copy of it has landed.  The root runs one plain GEMM launch, every other device ONE gated
// launch whose loaders wait inside the kernel (bounded) for the chunk count of their tile's rows.  All of it is
// built from the single-GPU entry points of this library (maize_chain_forward, maize_gemm_bf16_gated, ...), the
// same ones the one-process-per-GPU host path uses.
//
// One host thread per device enqueues that device's part of a step, so that the host cost of a step does not
// grow with the number of GPUs.  A call returns when everything is enqueued; maize_mgpu_sync waits and reports.
#include "../../include/maize_gemm.h"

#include <cuda_runtime.h>

#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int kFlagWords = 64;
constexpr int kFlagLanded = 16;  // word index: chunks of A that have landed on this device

struct StepArgs {
    int root = 0;
    const void *a_root = nullptr;
    uint32_t m = 0, n = 0, k = 0;
    void *const *a_local = nullptr;
    const void *const *b_shards = nullptr;
    void *const *c_shards = nullptr;
    uint64_t step = 0;        // steps run before this one
    uint32_t base = 0;        // chunk count before this step
    uint32_t chunk_rows = 0;
    bool a_on_stream = true;  // the root's forwarding waits for the root's compute stream as of the call
};

struct Rank {
    int device = -1;
    maize_ctx_t *ctx = nullptr;
    cudaStream_t compute = nullptr, push = nullptr;
    uint32_t *flags = nullptr;  // kFlagWords words in this device's memory
    // [step parity]: a step records the events of its own parity and waits for those of the other one, which the
    // previous step recorded; two sets, because another device's thread may already be recording this step's
    cudaEvent_t gemm_done[2] = {}, fwd_done[2] = {};
    cudaEvent_t entry = nullptr;
    // staging of the *_host entry point
    void *stage = nullptr;
    size_t stage_bytes = 0;
    // worker thread
    std::thread worker;
    std::mutex mu;
    std::condition_variable cv;
    bool has_task = false, done = false, quit = false;
    maize_status_t status = MAIZE_OK;
    std::string err;
};

}  // namespace

struct maize_mgpu {
    int n = 0;
    std::vector<Rank *> r;
    StepArgs args;
    uint32_t chunks_total = 0;
    uint64_t steps = 0;
    uint32_t chunk_rows = 2048;
    bool a_on_stream = true;
    std::string err;
};

namespace {

void shard_of(uint32_t n_rows, int world, int g, uint32_t *lo, uint32_t *hi)
{
    const uint32_t base = n_rows / world, extra = n_rows % world;
    const uint32_t ug = static_cast<uint32_t>(g);
    *lo = ug * base + (ug < extra ? ug : extra);
    *hi = *lo + base + (ug < extra ? 1u : 0u);
}

maize_status_t rank_fail(Rank &rk, maize_status_t st, const std::string &msg)
{
    rk.err = msg;
    return st;
}

// One device's part of a step; runs on that device's worker thread.
maize_status_t enqueue_step(maize_mgpu *mg, int g)
{
    Rank &rk = *mg->r[g];
    const StepArgs &s = mg->args;
    const int n = mg->n;
    const int pos = (g - s.root + n) % n;  // position in the chain
    const bool last = pos == n - 1;
    uint32_t lo, hi;
    shard_of(s.n, n, g, &lo, &hi);
    const uint32_t ns = hi - lo;
    cudaError_t e;
    if ((e = cudaSetDevice(rk.device)) != cudaSuccess)
        return rank_fail(rk, MAIZE_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    // The host runs at most two steps ahead of this device: the events of this parity were recorded two steps ago
    // and are about to be re-recorded.  (Deep queues of cross-device waits also measured slower.)
    if (s.step >= 2 && ((e = cudaEventSynchronize(rk.gemm_done[s.step & 1])) != cudaSuccess ||
                        (e = cudaEventSynchronize(rk.fwd_done[s.step & 1])) != cudaSuccess))
        return rank_fail(rk, MAIZE_ERR_CUDA, std::string("waiting for the step before last: ") + cudaGetErrorString(e));
    const uint64_t row_bytes = uint64_t(s.k) * 2;
    const void *a_here = pos == 0 ? s.a_root : s.a_local[g];
    maize_status_t st;
    if (!last && s.m > 0 && s.k > 0) {
        Rank &nx = *mg->r[(g + 1) % n];
        if (pos == 0 && s.a_on_stream) {
            // A may be the product of earlier work on the root's compute stream
            if ((e = cudaEventRecord(rk.entry, rk.compute)) != cudaSuccess ||
                (e = cudaStreamWaitEvent(rk.push, rk.entry, 0)) != cudaSuccess)
                return rank_fail(rk, MAIZE_ERR_CUDA, std::string("ordering the forwarding after A: ") + cudaGetErrorString(e));
        }
        // the next device's landing buffer is free once its GEMM and its own forwarding of the previous step are done
        if (s.step > 0 && ((e = cudaStreamWaitEvent(rk.push, nx.gemm_done[(s.step - 1) & 1], 0)) != cudaSuccess ||
                           (e = cudaStreamWaitEvent(rk.push, nx.fwd_done[(s.step - 1) & 1], 0)) != cudaSuccess))
            return rank_fail(rk, MAIZE_ERR_CUDA, std::string("waiting for the next device's buffer: ") + cudaGetErrorString(e));
        st = maize_chain_forward(rk.ctx, pos == 0 ? nullptr : rk.flags + kFlagLanded, s.base + 1, s.a_local[(g + 1) % n], a_here,
                                 uint64_t(s.m) * row_bytes, uint64_t(s.chunk_rows) * row_bytes, nx.flags + kFlagLanded, rk.push);
        if (st != MAIZE_OK)
            return rank_fail(rk, st, maize_last_error(rk.ctx));
    }
    if ((e = cudaEventRecord(rk.fwd_done[s.step & 1], rk.push)) != cudaSuccess)
        return rank_fail(rk, MAIZE_ERR_CUDA, std::string("cudaEventRecord: ") + cudaGetErrorString(e));
    if (ns > 0) {
        if (pos == 0)
            st = maize_gemm_bf16_ld(rk.ctx, a_here, s.k, s.b_shards[g], s.k, s.c_shards[g], ns, s.m, ns, s.k, rk.compute);
        else
            st = maize_gemm_bf16_gated(rk.ctx, a_here, s.k, s.b_shards[g], s.k, s.c_shards[g], ns, s.m, ns, s.k,
                                       rk.flags + kFlagLanded, s.base, s.chunk_rows, rk.compute);
        if (st != MAIZE_OK)
            return rank_fail(rk, st, maize_last_error(rk.ctx));
    }
    if ((e = cudaEventRecord(rk.gemm_done[s.step & 1], rk.compute)) != cudaSuccess)
        return rank_fail(rk, MAIZE_ERR_CUDA, std::string("cudaEventRecord: ") + cudaGetErrorString(e));
    return MAIZE_OK;
}

void worker_main(maize_mgpu *mg, int g)
{
    Rank &rk = *mg->r[g];
    cudaSetDevice(rk.device);
    for (;;) {
        std::unique_lock<std::mutex> lock(rk.mu);
        rk.cv.wait(lock, [&] { return rk.has_task || rk.quit; });
        if (rk.quit)
            return;
        rk.has_task = false;
        lock.unlock();
        const maize_status_t st = enqueue_step(mg, g);
        lock.lock();
        rk.status = st;
        rk.done = true;
        rk.cv.notify_all();
    }
}

maize_status_t mg_fail(maize_mgpu *mg, maize_status_t st, const std::string &msg)
{
    if (mg)
        mg->err = msg;
    return st;
}

void destroy_rank(Rank *rk)
{
    if (!rk)
        return;
    if (rk->worker.joinable()) {
        {
            std::lock_guard<std::mutex> lock(rk->mu);
            rk->quit = true;
        }
        rk->cv.notify_all();
        rk->worker.join();
    }
    if (rk->device >= 0)
        cudaSetDevice(rk->device);
    if (rk->compute)
        cudaStreamSynchronize(rk->compute);
    if (rk->push)
        cudaStreamSynchronize(rk->push);
    if (rk->ctx)
        maize_ctx_destroy(rk->ctx);
    if (rk->flags)
        cudaFree(rk->flags);
    if (rk->stage)
        cudaFree(rk->stage);
    for (cudaEvent_t ev : {rk->gemm_done[0], rk->gemm_done[1], rk->fwd_done[0], rk->fwd_done[1], rk->entry})
        if (ev)
            cudaEventDestroy(ev);
    if (rk->compute)
        cudaStreamDestroy(rk->compute);
    if (rk->push)
        cudaStreamDestroy(rk->push);
    delete rk;
}

}  // namespace

extern "C" {

maize_status_t maize_mgpu_create(int n, const int *devices, maize_mgpu_t **out)
{
    if (!out)
        return MAIZE_ERR_INVALID_ARG;
    *out = nullptr;
    if (n < 1 || n > 16 || !devices)
        return MAIZE_ERR_INVALID_ARG;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return MAIZE_ERR_NO_DEVICE;
    }
    for (int i = 0; i < n; ++i) {
        if (devices[i] < 0 || devices[i] >= count)
            return MAIZE_ERR_INVALID_ARG;
        for (int j = 0; j < i; ++j)
            if (devices[j] == devices[i])
                return MAIZE_ERR_INVALID_ARG;
    }
    int prev = -1;
    cudaGetDevice(&prev);
    maize_mgpu *mg = new (std::nothrow) maize_mgpu();
    if (!mg)
        return MAIZE_ERR_CUDA;
    mg->n = n;
    maize_status_t st = MAIZE_OK;
    for (int i = 0; i < n && st == MAIZE_OK; ++i) {
        Rank *rk = new (std::nothrow) Rank();
        if (!rk) {
            st = MAIZE_ERR_CUDA;
            break;
        }
        mg->r.push_back(rk);
        rk->device = devices[i];
        st = maize_ctx_create(devices[i], &rk->ctx);
        if (st != MAIZE_OK)
            break;
        bool ok = cudaSetDevice(devices[i]) == cudaSuccess;
        // every device reaches its chain successor's landing buffer and flag word directly
        for (int j = 0; ok && j < n; ++j) {
            if (j == i)
                continue;
            int can = 0;
            ok = cudaDeviceCanAccessPeer(&can, devices[i], devices[j]) == cudaSuccess && can;
            if (ok) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled)
                    cudaGetLastError();
                else
                    ok = e == cudaSuccess;
            }
        }
        ok = ok && cudaStreamCreateWithFlags(&rk->compute, cudaStreamNonBlocking) == cudaSuccess &&
             cudaStreamCreateWithFlags(&rk->push, cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&rk->gemm_done[0], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&rk->gemm_done[1], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&rk->fwd_done[0], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&rk->fwd_done[1], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&rk->entry, cudaEventDisableTiming) == cudaSuccess &&
             cudaMalloc(reinterpret_cast<void **>(&rk->flags), kFlagWords * sizeof(uint32_t)) == cudaSuccess &&
             cudaMemset(rk->flags, 0, kFlagWords * sizeof(uint32_t)) == cudaSuccess &&
             cudaDeviceSynchronize() == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            st = MAIZE_ERR_CUDA;
        }
    }
    if (st == MAIZE_OK) {
        for (int i = 0; i < n; ++i)
            mg->r[i]->worker = std::thread(worker_main, mg, i);
    }
    if (prev >= 0)
        cudaSetDevice(prev);
    if (st != MAIZE_OK) {
        maize_mgpu_destroy(mg);
        return st;
    }
    *out = mg;
    return MAIZE_OK;
}

void maize_mgpu_destroy(maize_mgpu_t *mg)
{
    if (!mg)
        return;
    int prev = -1;
    cudaGetDevice(&prev);
    for (Rank *rk : mg->r)
        destroy_rank(rk);
    if (prev >= 0)
        cudaSetDevice(prev);
    delete mg;
}

const char *maize_mgpu_last_error(const maize_mgpu_t *mg) { return mg ? mg->err.c_str() : "null handle"; }

int maize_mgpu_size(const maize_mgpu_t *mg) { return mg ? mg->n : 0; }

void *maize_mgpu_stream(const maize_mgpu_t *mg, int index)
{
    if (!mg || index < 0 || index >= mg->n)
        return nullptr;
    return mg->r[index]->compute;
}

maize_status_t maize_mgpu_shard(const maize_mgpu_t *mg, uint32_t n_rows, int index, uint32_t *first, uint32_t *end)
{
    if (!mg || index < 0 || index >= mg->n || !first || !end)
        return MAIZE_ERR_INVALID_ARG;
    shard_of(n_rows, mg->n, index, first, end);
    return MAIZE_OK;
}

maize_status_t maize_mgpu_set(maize_mgpu_t *mg, const char *key, int64_t value)
{
    if (!mg || !key)
        return MAIZE_ERR_INVALID_ARG;
    if (!strcmp(key, "chunk_rows")) {
        if (value < 256 || value > (1 << 24) || value % 256 != 0)
            return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "chunk_rows: a multiple of 256");
        mg->chunk_rows = static_cast<uint32_t>(value);
    } else if (!strcmp(key, "a_on_stream")) {
        mg->a_on_stream = value != 0;
    } else {
        // everything else goes to the per-device contexts (timeout_ns, chain_streams, ...)
        for (Rank *rk : mg->r) {
            const maize_status_t st = maize_ctx_set(rk->ctx, key, value);
            if (st != MAIZE_OK)
                return mg_fail(mg, st, maize_last_error(rk->ctx));
        }
    }
    return MAIZE_OK;
}

maize_status_t maize_gemm_bf16_nsharded(maize_mgpu_t *mg, int root, const void *a_on_root, uint32_t m, uint32_t k,
                                        void *const *a_local, const void *const *b_shards, uint32_t n,
                                        void *const *c_shards)
{
    if (!mg)
        return MAIZE_ERR_INVALID_ARG;
    mg->err.clear();
    if (root < 0 || root >= mg->n)
        return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "root is not an index into the device list");
    if (m == 0 || n == 0)
        return MAIZE_OK;
    if (!b_shards || !c_shards || (mg->n > 1 && !a_local) || (!a_on_root && k > 0))
        return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "null pointer array or null A");
    if (k % 8 != 0)
        return mg_fail(mg, MAIZE_ERR_UNSUPPORTED, "K must be a multiple of 8 (16-byte TMA row pitch)");
    for (int g = 0; g < mg->n; ++g) {
        uint32_t lo, hi;
        shard_of(n, mg->n, g, &lo, &hi);
        if (hi > lo && (!c_shards[g] || (!b_shards[g] && k > 0)))
            return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "null shard pointer");
        if (g != root && !a_local[g] && k > 0)
            return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "null landing buffer for a device other than the root");
    }
    StepArgs &s = mg->args;
    s.root = root;
    s.a_root = a_on_root;
    s.m = m;
    s.n = n;
    s.k = k;
    s.a_local = a_local;
    s.b_shards = b_shards;
    s.c_shards = c_shards;
    s.step = mg->steps;
    s.base = mg->chunks_total;
    s.chunk_rows = mg->chunk_rows;
    s.a_on_stream = mg->a_on_stream;
    // every device enqueues its own part on its own thread
    for (Rank *rk : mg->r) {
        std::lock_guard<std::mutex> lock(rk->mu);
        rk->done = false;
        rk->has_task = true;
        rk->cv.notify_all();
    }
    maize_status_t st = MAIZE_OK;
    for (Rank *rk : mg->r) {
        std::unique_lock<std::mutex> lock(rk->mu);
        rk->cv.wait(lock, [&] { return rk->done; });
        if (rk->status != MAIZE_OK && st == MAIZE_OK) {
            st = rk->status;
            char buf[64];
            snprintf(buf, sizeof buf, "device %d: ", rk->device);
            mg->err = std::string(buf) + rk->err;
        }
    }
    mg->chunks_total += (m + mg->chunk_rows - 1) / mg->chunk_rows;
    mg->steps += 1;
    return st;
}

maize_status_t maize_mgpu_sync(maize_mgpu_t *mg)
{
    if (!mg)
        return MAIZE_ERR_INVALID_ARG;
    int prev = -1;
    cudaGetDevice(&prev);
    maize_status_t st = MAIZE_OK;
    for (Rank *rk : mg->r) {
        cudaSetDevice(rk->device);
        cudaError_t e = cudaStreamSynchronize(rk->push);
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(rk->compute);
        maize_status_t here = e == cudaSuccess ? maize_ctx_poll(rk->ctx, rk->compute) : MAIZE_ERR_CUDA;
        if (here != MAIZE_OK && st == MAIZE_OK) {
            st = here;
            char buf[64];
            snprintf(buf, sizeof buf, "device %d: ", rk->device);
            mg->err = std::string(buf) + (e == cudaSuccess ? maize_last_error(rk->ctx) : cudaGetErrorString(e));
        }
    }
    if (prev >= 0)
        cudaSetDevice(prev);
    return st;
}

maize_status_t maize_gemm_bf16_nsharded_host(maize_mgpu_t *mg, int root, const void *a_host, uint32_t m, uint32_t k,
                                             const void *b_host, uint32_t n, void *c_host)
{
    if (!mg)
        return MAIZE_ERR_INVALID_ARG;
    mg->err.clear();
    if (root < 0 || root >= mg->n)
        return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "root is not an index into the device list");
    if (m == 0 || n == 0)
        return MAIZE_OK;
    if (!c_host || ((!a_host || !b_host) && k > 0))
        return mg_fail(mg, MAIZE_ERR_INVALID_ARG, "null host pointer");
    if (k % 8 != 0)
        return mg_fail(mg, MAIZE_ERR_UNSUPPORTED, "K must be a multiple of 8 (16-byte TMA row pitch)");
    int prev = -1;
    cudaGetDevice(&prev);
    auto round_up = [](size_t x) { return (x + 255) & ~size_t(255); };
    std::vector<void *> a_local(mg->n), c_sh(mg->n);
    std::vector<const void *> b_sh(mg->n);
    const size_t a_bytes = round_up(size_t(m) * k * 2);
    maize_status_t st = MAIZE_OK;
    for (int g = 0; g < mg->n && st == MAIZE_OK; ++g) {
        Rank &rk = *mg->r[g];
        uint32_t lo, hi;
        shard_of(n, mg->n, g, &lo, &hi);
        const size_t b_bytes = round_up(size_t(hi - lo) * k * 2), c_bytes = round_up(size_t(m) * (hi - lo) * 2);
        const size_t need = a_bytes + b_bytes + c_bytes + 256;
        cudaSetDevice(rk.device);
        if (need > rk.stage_bytes) {
            // the staging of a device grows on demand, like that of maize_gemm_bf16_host
            cudaStreamSynchronize(rk.compute);
            cudaStreamSynchronize(rk.push);
            if (rk.stage)
                cudaFree(rk.stage);
            rk.stage = nullptr;
            rk.stage_bytes = 0;
            const cudaError_t e = cudaMalloc(&rk.stage, need);
            if (e != cudaSuccess) {
                st = mg_fail(mg, MAIZE_ERR_CUDA, std::string("cudaMalloc(staging): ") + cudaGetErrorString(e));
                break;
            }
            rk.stage_bytes = need;
        }
        char *base = static_cast<char *>(rk.stage);
        a_local[g] = base;
        b_sh[g] = base + a_bytes;
        c_sh[g] = base + a_bytes + b_bytes;
        cudaError_t e = cudaSuccess;
        if (g == root && k > 0)
            e = cudaMemcpyAsync(base, a_host, size_t(m) * k * 2, cudaMemcpyHostToDevice, rk.compute);
        if (e == cudaSuccess && hi > lo && k > 0)
            e = cudaMemcpyAsync(base + a_bytes, static_cast<const char *>(b_host) + size_t(lo) * k * 2,
                                size_t(hi - lo) * k * 2, cudaMemcpyHostToDevice, rk.compute);
        if (e != cudaSuccess)
            st = mg_fail(mg, MAIZE_ERR_CUDA, std::string("H2D copy: ") + cudaGetErrorString(e));
    }
    if (st == MAIZE_OK) {
        const bool keep = mg->a_on_stream;
        mg->a_on_stream = true;  // A reaches the root on its compute stream
        st = maize_gemm_bf16_nsharded(mg, root, a_local[root], m, k, a_local.data(), b_sh.data(), n, c_sh.data());
        mg->a_on_stream = keep;
    }
    for (int g = 0; g < mg->n && st == MAIZE_OK; ++g) {
        Rank &rk = *mg->r[g];
        uint32_t lo, hi;
        shard_of(n, mg->n, g, &lo, &hi);
        if (hi == lo)
            continue;
        cudaSetDevice(rk.device);
        // column block [lo, hi) of the dense host C
        const cudaError_t e = cudaMemcpy2DAsync(static_cast<char *>(c_host) + size_t(lo) * 2, size_t(n) * 2, c_sh[g],
                                                size_t(hi - lo) * 2, size_t(hi - lo) * 2, m, cudaMemcpyDeviceToHost,
                                                rk.compute);
        if (e != cudaSuccess)
            st = mg_fail(mg, MAIZE_ERR_CUDA, std::string("D2H copy: ") + cudaGetErrorString(e));
    }
    if (prev >= 0)
        cudaSetDevice(prev);
    const maize_status_t waited = maize_mgpu_sync(mg);
    return st != MAIZE_OK ? st : waited;
}

}  // extern "C"
