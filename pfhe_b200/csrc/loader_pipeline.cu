// Staged loader: packed GGUF bytes in ordinary host memory (or in a file)
// -> pinned ring slot (host threads) -> device slot (cudaMemcpyAsync on a copy
// stream) -> decode kernel on the caller's stream.  The transfer of chunk i+1
// overlaps the decode of chunk i; slot reuse is gated by events.  This replaces
// the host-to-device leg of GGUFReader.read_tensor in the reference
// (src/phfe/inference/gguf_loader.py:356 and :378), which copies already
// dequantised fp32 data from pageable memory synchronously.
#include "common.h"
#include "host_copy.h"

#include <errno.h>
#include <stdlib.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace pfhe {
namespace {

using Clock = std::chrono::steady_clock;
inline double seconds_since(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

// Fixed pool that runs one indexed job at a time across all workers plus the
// caller.  Indices are handed out under the mutex (the jobs are multi-megabyte
// copies, so the lock is never contended for long).
class CopyPool {
public:
    explicit CopyPool(int n_threads) {
        for (int i = 0; i < n_threads; ++i) workers_.emplace_back([this] { worker(); });
    }
    ~CopyPool() {
        { std::lock_guard<std::mutex> lk(mu_); stop_ = true; }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    // Runs fn(i) for i in [0, n); returns when all are done.
    void run(int n, const std::function<void(int)> &fn) {
        if (n <= 0) return;
        if (workers_.empty() || n == 1) { for (int i = 0; i < n; ++i) fn(i); return; }
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &fn; total_ = n; next_ = 0; pending_ = n;
            generation_.fetch_add(1, std::memory_order_release);
        }
        cv_.notify_all();
        drain();
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [this] { return pending_ == 0; });
        fn_ = nullptr; total_ = 0; next_ = 0;
    }

private:
    // Takes indices until none are left; returns with the lock released.
    void drain() {
        std::unique_lock<std::mutex> lk(mu_);
        while (fn_ && next_ < total_) {
            const int i = next_++;
            const std::function<void(int)> *fn = fn_;
            lk.unlock();
            (*fn)(i);
            lk.lock();
            if (--pending_ == 0) done_cv_.notify_all();
        }
    }
    void worker() {
        unsigned seen = 0;
        for (;;) {
            // During a load the next job follows the last within tens of microseconds: watch for it
            // for a moment before sleeping, which saves the wake-up latency of the condition variable.
            const auto t0 = Clock::now();
            while (generation_.load(std::memory_order_acquire) == seen && seconds_since(t0) < 100e-6) {
#if defined(__x86_64__)
                __builtin_ia32_pause();
#endif
            }
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || (fn_ && next_ < total_); });
                if (stop_) return;
                seen = generation_.load(std::memory_order_relaxed);
            }
            drain();
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    const std::function<void(int)> *fn_ = nullptr;
    int next_ = 0, total_ = 0, pending_ = 0;
    std::atomic<unsigned> generation_{0};   // bumped for every job; lets idle workers notice one without the lock
    bool stop_ = false;
};

struct Slot {
    uint8_t *pinned = nullptr;
    uint8_t *dev = nullptr;
    cudaEvent_t copied = nullptr;   // H2D finished (copy stream)
    cudaEvent_t done = nullptr;     // decode that read the slot finished (caller stream)
    bool in_use = false;
};

// Polls an event until it completes or the deadline passes.
int wait_event_bounded(cudaEvent_t ev, int timeout_ms, const char *what)
{
    const auto t0 = Clock::now();
    for (int spin = 0;; ++spin) {
        cudaError_t e = cudaEventQuery(ev);
        if (e == cudaSuccess) return PFHE_OK;
        if (e != cudaErrorNotReady) return cuda_fail(e, what);
        if (timeout_ms >= 0 && seconds_since(t0) * 1e3 > timeout_ms) {
            set_error("%s: not finished after %d ms", what, timeout_ms);
            return PFHE_ERR_TIMEOUT;
        }
        if (spin > 200) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    int enter(int dev) {
        cudaError_t e = cudaGetDevice(&prev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
        if (prev != dev) {
            e = cudaSetDevice(dev);
            if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
            changed = true;
        }
        return PFHE_OK;
    }
    ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

}  // namespace
}  // namespace pfhe

using namespace pfhe;

struct pfhe_loader {
    int device = 0;
    int64_t slot_bytes = 0;
    std::vector<Slot> slots;
    int next_slot = 0;
    cudaStream_t copy_stream = nullptr;
    CopyPool *pool = nullptr;
    int n_threads = 1;                   // copy threads including the submitting one
    pfhe_loader_stats stats{};
    std::mutex mu;                       // one submit at a time per loader
    bool streaming_copy = true;          // non-temporal stores into the pinned slots
    int slot_timeout_ms = 120000;
};

namespace {

// Host copy granularity per worker job: about eight pieces per thread and chunk, so that the
// threads finish a chunk within one short piece of each other (with fixed 2 MiB pieces a 64 MiB
// chunk is 32 jobs for 12 threads: a third of them idle through the last round), between 64 KiB
// and 2 MiB, a multiple of 4 KiB.
int64_t copy_piece_bytes(int64_t bytes, int n_threads)
{
    int64_t piece = bytes / ((int64_t)(n_threads > 0 ? n_threads : 1) * 8);
    if (piece < (64 << 10)) piece = 64 << 10;
    if (piece > (2 << 20)) piece = 2 << 20;
    return (piece + 4095) & ~(int64_t)4095;
}

struct Source {
    const uint8_t *host = nullptr;       // when non-null: memcpy source
    int fd = -1;                         // otherwise pread source
    int64_t file_offset = 0;
};

int fill_pinned(pfhe_loader *ld, uint8_t *dst, const Source &src, int64_t offset, int64_t bytes)
{
    const int64_t piece = copy_piece_bytes(bytes, ld->n_threads);
    const int pieces = (int)((bytes + piece - 1) / piece);
    std::atomic<int> io_errno{0};
    ld->pool->run(pieces, [&](int i) {
        const int64_t a = (int64_t)i * piece;
        const int64_t n = (bytes - a) < piece ? (bytes - a) : piece;
        if (src.host) {
            copy_to_pinned(dst + a, src.host + offset + a, (size_t)n, ld->streaming_copy);
        } else {
            int64_t got = 0;
            while (got < n) {
                const ssize_t r = pread(src.fd, dst + a + got, (size_t)(n - got), (off_t)(src.file_offset + offset + a + got));
                if (r < 0) { if (errno == EINTR) continue; io_errno.store(errno); return; }
                if (r == 0) { io_errno.store(ENODATA); return; }
                got += r;
            }
        }
    });
    if (io_errno.load()) { set_error("pread failed: %s", strerror(io_errno.load())); return PFHE_ERR_BAD_ARG; }
    return PFHE_OK;
}

int submit_impl(pfhe_loader *ld, const Source &src, int64_t src_bytes, int ggml_type, int mid, int out, void *dst_dev,
                int64_t dst_bytes, int64_t n_elements, cudaStream_t stream)
{
    if (!ld) { set_error("null loader"); return PFHE_ERR_BAD_ARG; }
    int be = 0, bb = 0;
    int rc = type_geometry(ggml_type, &be, &bb);
    if (rc) return rc;
    const int osz = out_size(out);
    if (osz == 0 || out_size(mid) == 0) { set_error("output dtype %d / intermediate dtype %d not in {f32,f16,bf16}", out, mid); return PFHE_ERR_BAD_DTYPE; }
    if (n_elements < 0 || src_bytes < 0 || dst_bytes < 0) { set_error("negative size"); return PFHE_ERR_BAD_ARG; }
    const int64_t need = (n_elements + be - 1) / be * bb;
    if (src_bytes < need) { set_error("Data too short: %lld < %lld", (long long)src_bytes, (long long)need); return PFHE_ERR_SHORT_SOURCE; }
    if (dst_bytes < n_elements * osz) { set_error("destination too small: %lld < %lld", (long long)dst_bytes, (long long)(n_elements * osz)); return PFHE_ERR_SHORT_DEST; }
    if (n_elements == 0) return PFHE_OK;
    if (!dst_dev || (!src.host && src.fd < 0)) { set_error("null pointer"); return PFHE_ERR_BAD_ARG; }

    std::lock_guard<std::mutex> lk(ld->mu);
    DeviceGuard guard;
    if ((rc = guard.enter(ld->device))) return rc;

    // Chunks hold whole 8-block groups (block formats) or multiples of 16
    // elements, so every chunk starts on a 16-byte line on both sides.
    int64_t chunk_elems;
    if (be > 1) chunk_elems = ld->slot_bytes / (8 * bb) * 8 * be;
    else chunk_elems = ld->slot_bytes / bb / 16 * 16;
    if (chunk_elems <= 0) { set_error("slot too small"); return PFHE_ERR_BAD_ARG; }

    ld->stats.tensors++;
    for (int64_t e0 = 0; e0 < n_elements; e0 += chunk_elems) {
        const int64_t ne = (n_elements - e0) < chunk_elems ? (n_elements - e0) : chunk_elems;
        const int64_t off = e0 / be * bb;
        const int64_t nb = (ne + be - 1) / be * bb;
        Slot &s = ld->slots[ld->next_slot];
        ld->next_slot = (ld->next_slot + 1) % (int)ld->slots.size();
        if (s.in_use) {
            const auto t0 = Clock::now();
            rc = wait_event_bounded(s.done, ld->slot_timeout_ms, "waiting for a free staging slot");
            ld->stats.slot_wait_seconds += seconds_since(t0);
            if (rc) return rc;
        }
        const auto t0 = Clock::now();
        if ((rc = fill_pinned(ld, s.pinned, src, off, nb))) return rc;
        ld->stats.host_copy_seconds += seconds_since(t0);

        cudaError_t e = cudaMemcpyAsync(s.dev, s.pinned, (size_t)nb, cudaMemcpyHostToDevice, ld->copy_stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(H2D)");
        if ((e = cudaEventRecord(s.copied, ld->copy_stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord(copied)");
        if ((e = cudaStreamWaitEvent(stream, s.copied, 0)) != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
        rc = launch_decode(ggml_type, mid, out, s.dev, nb, static_cast<uint8_t *>(dst_dev) + e0 * osz, ne * osz, ne, stream, nullptr);
        if (rc) return rc;
        if ((e = cudaEventRecord(s.done, stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord(done)");
        s.in_use = true;
        ld->stats.bytes_staged += nb;
        ld->stats.bytes_decoded += ne * osz;
        ld->stats.chunks++;
    }
    return PFHE_OK;
}

}  // namespace

extern "C" {

int pfhe_loader_create(int device, int n_slots, int64_t slot_bytes, int n_threads, pfhe_loader **out)
{
    if (!out || n_slots < 1 || n_slots > 64 || slot_bytes < 8 * 34 * 4) { set_error("bad loader arguments"); return PFHE_ERR_BAD_ARG; }
    *out = nullptr;
    DeviceGuard guard;
    int rc = guard.enter(device);
    if (rc) return rc;
    pfhe_loader *ld = new pfhe_loader();
    ld->device = device;
    ld->slot_bytes = (slot_bytes + 255) & ~(int64_t)255;
    cudaError_t e = cudaStreamCreateWithFlags(&ld->copy_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete ld; return cuda_fail(e, "cudaStreamCreate"); }
    ld->slots.resize(n_slots);
    for (auto &s : ld->slots) {
        void *p = nullptr;
        if ((e = cudaHostAlloc(&p, (size_t)ld->slot_bytes, cudaHostAllocPortable)) != cudaSuccess) break;
        s.pinned = static_cast<uint8_t *>(p);
        if ((e = cudaMalloc(&p, (size_t)ld->slot_bytes + 256)) != cudaSuccess) break;
        s.dev = static_cast<uint8_t *>(p);
        if ((e = cudaEventCreateWithFlags(&s.copied, cudaEventDisableTiming)) != cudaSuccess) break;
        if ((e = cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming)) != cudaSuccess) break;
    }
    if (e != cudaSuccess) {
        rc = cuda_fail(e, "allocating staging slots");
        pfhe_loader_destroy(ld);
        return rc;
    }
    if (n_threads <= 0) {
        unsigned hc = std::thread::hardware_concurrency();
        n_threads = hc >= 32 ? 8 : (hc >= 8 ? 4 : 2);
    }
    if (const char *mode = getenv("PFHE_HOST_COPY")) ld->streaming_copy = strcmp(mode, "memcpy") != 0;
    ld->n_threads = n_threads;
    ld->pool = new CopyPool(n_threads - 1);
    *out = ld;
    return PFHE_OK;
}

int pfhe_loader_submit(pfhe_loader *ld, const void *host_src, int64_t src_bytes, int ggml_type, int mid_dtype,
                       int out_dtype, void *dst_dev, int64_t dst_bytes, int64_t n_elements, void *stream)
{
    Source s;
    s.host = static_cast<const uint8_t *>(host_src);
    if (!host_src && n_elements > 0) { set_error("null host source"); return PFHE_ERR_BAD_ARG; }
    return submit_impl(ld, s, src_bytes, ggml_type, mid_dtype, out_dtype, dst_dev, dst_bytes, n_elements,
                       static_cast<cudaStream_t>(stream));
}

int pfhe_loader_submit_fd(pfhe_loader *ld, int fd, int64_t file_offset, int64_t src_bytes, int ggml_type,
                          int mid_dtype, int out_dtype, void *dst_dev, int64_t dst_bytes, int64_t n_elements,
                          void *stream)
{
    Source s;
    s.fd = fd;
    s.file_offset = file_offset;
    if (fd < 0 || file_offset < 0) { set_error("bad file descriptor or offset"); return PFHE_ERR_BAD_ARG; }
    return submit_impl(ld, s, src_bytes, ggml_type, mid_dtype, out_dtype, dst_dev, dst_bytes, n_elements,
                       static_cast<cudaStream_t>(stream));
}

int pfhe_loader_upload(pfhe_loader *ld, const void *host_src, int64_t bytes, void *dst_dev, void *stream_)
{
    if (!ld) { set_error("null loader"); return PFHE_ERR_BAD_ARG; }
    if (bytes < 0) { set_error("negative size"); return PFHE_ERR_BAD_ARG; }
    if (bytes == 0) return PFHE_OK;
    if (!host_src || !dst_dev) { set_error("null pointer"); return PFHE_ERR_BAD_ARG; }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    std::lock_guard<std::mutex> lk(ld->mu);
    DeviceGuard guard;
    int rc = guard.enter(ld->device);
    if (rc) return rc;
    Source src;
    src.host = static_cast<const uint8_t *>(host_src);
    ld->stats.tensors++;
    for (int64_t off = 0; off < bytes; off += ld->slot_bytes) {
        const int64_t nb = (bytes - off) < ld->slot_bytes ? (bytes - off) : ld->slot_bytes;
        Slot &s = ld->slots[ld->next_slot];
        ld->next_slot = (ld->next_slot + 1) % (int)ld->slots.size();
        if (s.in_use) {
            const auto t0 = Clock::now();
            rc = wait_event_bounded(s.done, ld->slot_timeout_ms, "waiting for a free staging slot");
            ld->stats.slot_wait_seconds += seconds_since(t0);
            if (rc) return rc;
        }
        const auto t0 = Clock::now();
        if ((rc = fill_pinned(ld, s.pinned, src, off, nb))) return rc;
        ld->stats.host_copy_seconds += seconds_since(t0);
        // pinned slot -> destination directly: the packed bytes are the result, no device staging
        cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t *>(dst_dev) + off, s.pinned, (size_t)nb, cudaMemcpyHostToDevice,
                                        ld->copy_stream);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(H2D)");
        if ((e = cudaEventRecord(s.done, ld->copy_stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord(done)");
        if ((e = cudaStreamWaitEvent(stream, s.done, 0)) != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
        s.in_use = true;
        ld->stats.bytes_staged += nb;
        ld->stats.chunks++;
    }
    return PFHE_OK;
}

int pfhe_loader_wait(pfhe_loader *ld, int timeout_ms)
{
    if (!ld) { set_error("null loader"); return PFHE_ERR_BAD_ARG; }
    std::lock_guard<std::mutex> lk(ld->mu);
    DeviceGuard guard;
    int rc = guard.enter(ld->device);
    if (rc) return rc;
    for (auto &s : ld->slots) {
        if (!s.in_use) continue;
        if ((rc = wait_event_bounded(s.done, timeout_ms, "waiting for queued decodes"))) return rc;
        s.in_use = false;
    }
    return pfhe_device_status(ld->device);
}

int pfhe_loader_get_stats(pfhe_loader *ld, pfhe_loader_stats *out)
{
    if (!ld || !out) { set_error("null argument"); return PFHE_ERR_BAD_ARG; }
    std::lock_guard<std::mutex> lk(ld->mu);
    *out = ld->stats;
    return PFHE_OK;
}

int pfhe_loader_destroy(pfhe_loader *ld)
{
    if (!ld) return PFHE_OK;
    DeviceGuard guard;
    int rc = guard.enter(ld->device);
    if (rc == PFHE_OK) {
        for (auto &s : ld->slots)
            if (s.in_use && s.done) (void)wait_event_bounded(s.done, 30000, "draining loader");
    }
    delete ld->pool;
    for (auto &s : ld->slots) {
        if (s.copied) cudaEventDestroy(s.copied);
        if (s.done) cudaEventDestroy(s.done);
        if (s.dev) cudaFree(s.dev);
        if (s.pinned) cudaFreeHost(s.pinned);
    }
    if (ld->copy_stream) cudaStreamDestroy(ld->copy_stream);
    delete ld;
    return PFHE_OK;
}

}  // extern "C"
