// BFCKPT1 files (include/blackforge/backend/cpu/checkpoint.hpp:15-24: magic "BFCKPT1\0", u32 tensor count, then per
// tensor u32 name length, name, u32 rank, u64 dims, fp32 data, all little-endian), read as a stream.
//
// The reference's loader (src/backend/cuda/checkpoint.cu:82-130) reads every tensor whole into a host vector and
// uploads it with a synchronous copy. At the sizes this backend is built for (97 GB of fp32 for the 24B-class
// configuration, 12 GB of it per rank under 8-way tensor parallelism) that means a pageable staging copy as large
// as the largest tensor and no overlap between the disk and the bus. Here:
//   1. an index pass reads the headers only (pread, no data) and checks the file's extent against every tensor;
//   2. names and shapes are checked against the model before a single byte is uploaded;
//   3. reader threads pread whole rows into a ring of pinned buffers, only the rows this tensor-parallel rank
//      holds for row-sharded tensors, while the calling thread issues the asynchronous uploads (a strided copy
//      takes this rank's columns out of full rows for column-sharded tensors). Pieces of a few MiB keep a piece in
//      the CPU's caches between the read and the copy engine's fetch (with four readers, 2-4 MiB pieces load 1.6x faster than 16 MiB ones).
// The on-disk format is unchanged; saveCheckpoint writes files the reference reads.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>
#include <map>
#include <mutex>
#include <thread>

#include "../common.cuh"
#include "bfb200.hpp"

namespace bfb200 {

using bfb::fail;

namespace {

constexpr char kMagic[8] = {'B', 'F', 'C', 'K', 'P', 'T', '1', '\0'};
[[noreturn]] void ioFail(const std::string& text) { fail(BFB_IO_ERROR, text); }

struct Fd {
    int fd = -1;
    explicit Fd(const std::string& path) : fd(::open(path.c_str(), O_RDONLY | O_CLOEXEC)) {}
    ~Fd() {
        if (fd >= 0) ::close(fd);
    }
    Fd(const Fd&) = delete;
    Fd& operator=(const Fd&) = delete;
};

// pread until `bytes` are in or the file ends; returns what was read
std::size_t readAt(int fd, void* dst, std::size_t bytes, std::uint64_t offset) {
    std::size_t done = 0;
    while (done < bytes) {
        const ssize_t got = ::pread(fd, static_cast<char*>(dst) + done, bytes - done, static_cast<off_t>(offset + done));
        if (got < 0) {
            if (errno == EINTR) continue;
            return done;
        }
        if (got == 0) break;
        done += static_cast<std::size_t>(got);
    }
    return done;
}

struct Segment {
    std::size_t param = 0;
    std::size_t firstRow = 0, rows = 0;
    std::uint64_t offset = 0;
    std::size_t bytes = 0;
    void* deviceDst = nullptr;   // pieces of a converted-weights file go straight to this address
};

// Pinned staging buffers that travel between the reader thread and the uploading thread.
class Ring {
public:
    Ring(int count, std::size_t bytes) {
        for (int i = 0; i < count; ++i) {
            void* p = nullptr;
            if (cudaMallocHost(&p, bytes) != cudaSuccess) {
                (void)cudaGetLastError();
                release();
                fail(BFB_CUDA_ERROR, "loadCheckpoint: cannot allocate pinned staging memory");
            }
            buffers_.push_back(p);
            free_.push_back(i);
        }
    }
    ~Ring() { release(); }
    void* data(int i) const { return buffers_[static_cast<std::size_t>(i)]; }

    int takeFree() {   // reader side; -1 once the load was abandoned
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [&] { return !free_.empty() || stop_; });
        if (stop_) return -1;
        const int i = free_.front();
        free_.pop_front();
        return i;
    }
    void giveFree(int i) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            free_.push_back(i);
        }
        cv_.notify_all();
    }
    void giveFilled(int i, const Segment& s) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            filled_.push_back({i, s});
        }
        cv_.notify_all();
    }
    // uploader side; false when the reader is done (or failed) and nothing is left
    bool takeFilled(int* i, Segment* s) {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [&] { return !filled_.empty() || readerDone_; });
        if (filled_.empty()) return false;
        *i = filled_.front().first;
        *s = filled_.front().second;
        filled_.pop_front();
        return true;
    }
    void setReaders(int count) { readersLeft_ = count; }
    void readerFinished(const std::string& error) {
        {
            std::lock_guard<std::mutex> lock(mu_);
            if (--readersLeft_ <= 0) readerDone_ = true;
            if (!error.empty()) {
                if (error_.empty()) error_ = error;
                stop_ = true;   // the other readers stop at their next buffer
            }
        }
        cv_.notify_all();
    }
    void abandon() {
        {
            std::lock_guard<std::mutex> lock(mu_);
            stop_ = true;
        }
        cv_.notify_all();
    }
    std::string error() {
        std::lock_guard<std::mutex> lock(mu_);
        return error_;
    }

private:
    void release() {
        for (void* p : buffers_) cudaFreeHost(p);
        buffers_.clear();
    }
    std::vector<void*> buffers_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<int> free_;
    std::deque<std::pair<int, Segment>> filled_;
    int readersLeft_ = 1;
    bool readerDone_ = false, stop_ = false;
    std::string error_;
};

// Reads the pieces with a few threads into pinned buffers while the calling thread hands each filled buffer to `upload`
// (which issues asynchronous copies on the given stream and returns the bytes it sent). Returns their sum.
using UploadFn = std::function<std::size_t(const Segment&, const void*, cudaStream_t)>;
std::size_t streamSegments(const std::string& path, const std::vector<Segment>& segments, std::size_t largest,
                           const UploadFn& upload) {
    std::size_t uploadedBytes = 0;
    Fd file(path);
    if (file.fd < 0) ioFail("loadCheckpoint: cannot open '" + path + "'");
    // a few readers (pread is thread-safe and the pieces are independent); two more buffers than readers, so that
    // uploads are in flight while every reader holds one
    const int readers = static_cast<int>(std::max<std::size_t>(
        1, std::min<std::size_t>({4, segments.size(), std::max(1u, std::thread::hardware_concurrency() / 2)})));
    const int kBuffers = readers + 2;
    Ring ring(kBuffers, largest);
    ring.setReaders(readers);
    cudaStream_t stream = nullptr;
    BFB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    std::vector<cudaEvent_t> uploaded(static_cast<std::size_t>(kBuffers), nullptr);
    for (auto& e : uploaded) BFB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));

    std::atomic<std::size_t> nextSegment{0};
    std::vector<std::thread> readerThreads;
    for (int t = 0; t < readers; ++t) {
        readerThreads.emplace_back([&] {
            std::string error;
            while (true) {
                const std::size_t i = nextSegment.fetch_add(1);
                if (i >= segments.size()) break;
                const Segment& s = segments[i];
                const int b = ring.takeFree();
                if (b < 0) break;
                if (readAt(file.fd, ring.data(b), s.bytes, s.offset) != s.bytes) {
                    error = "loadCheckpoint: '" + path + "' is truncated or corrupt";
                    break;
                }
                ring.giveFilled(b, s);
            }
            ring.readerFinished(error);
        });
    }

    std::string failure;
    try {
        std::deque<int> inFlight;
        int b = 0;
        Segment s;
        while (ring.takeFilled(&b, &s)) {
            uploadedBytes += upload(s, ring.data(b), stream);
            BFB_CUDA(cudaEventRecord(uploaded[b], stream));
            inFlight.push_back(b);
            while (inFlight.size() >= 2) {   // the other buffers stay with the readers
                BFB_CUDA(cudaEventSynchronize(uploaded[inFlight.front()]));
                ring.giveFree(inFlight.front());
                inFlight.pop_front();
            }
        }
        BFB_CUDA(cudaStreamSynchronize(stream));
    } catch (const std::exception& e) {
        failure = e.what();
    }
    ring.abandon();
    for (std::thread& t : readerThreads) t.join();
    (void)cudaStreamSynchronize(stream);
    for (auto& e : uploaded) cudaEventDestroy(e);
    cudaStreamDestroy(stream);
    if (!failure.empty()) fail(BFB_CUDA_ERROR, failure);
    if (!ring.error().empty()) ioFail(ring.error());
    return uploadedBytes;
}

}  // namespace

std::vector<CheckpointEntry> indexCheckpoint(const std::string& path) {
    Fd file(path);
    if (file.fd < 0) ioFail("loadCheckpoint: cannot open '" + path + "'");
    struct stat st {};
    if (::fstat(file.fd, &st) != 0) ioFail("loadCheckpoint: cannot stat '" + path + "'");
    const std::uint64_t size = static_cast<std::uint64_t>(st.st_size);
    std::uint64_t at = 0;
    auto take = [&](void* dst, std::size_t bytes, const char* what) {
        if (at + bytes > size || readAt(file.fd, dst, bytes, at) != bytes) {
            ioFail("loadCheckpoint: '" + path + "' is truncated" + (what[0] != '\0' ? std::string(" or corrupt (") + what + ")" : ""));
        }
        at += bytes;
    };
    char magic[8];
    if (size < sizeof(magic) || readAt(file.fd, magic, sizeof(magic), 0) != sizeof(magic) ||
        std::memcmp(magic, kMagic, sizeof(kMagic)) != 0) {
        ioFail("loadCheckpoint: '" + path + "' is not a BlackForge checkpoint");
    }
    at = sizeof(magic);
    std::uint32_t count = 0;
    take(&count, sizeof(count), "");
    std::vector<CheckpointEntry> entries;
    entries.reserve(std::min<std::uint32_t>(count, 1u << 16));
    for (std::uint32_t i = 0; i < count; ++i) {
        CheckpointEntry e;
        std::uint32_t nameLen = 0, rank = 0;
        take(&nameLen, sizeof(nameLen), "name length");
        if (nameLen > (1u << 20)) ioFail("loadCheckpoint: '" + path + "' is truncated or corrupt (name length)");
        e.name.resize(nameLen);
        take(e.name.data(), nameLen, "name");
        take(&rank, sizeof(rank), "rank");
        if (rank > 8) ioFail("loadCheckpoint: '" + path + "' is truncated or corrupt (rank)");
        std::uint64_t elements = 1;
        for (std::uint32_t d = 0; d < rank; ++d) {
            std::uint64_t dim = 0;
            take(&dim, sizeof(dim), "shape");
            if (dim != 0 && elements > (std::uint64_t(1) << 62) / dim) {
                ioFail("loadCheckpoint: '" + path + "' is truncated or corrupt (shape)");
            }
            elements *= dim;
            e.shape.push_back(static_cast<std::size_t>(dim));
        }
        e.dataOffset = at;
        e.dataBytes = elements * sizeof(float);
        if (e.dataBytes > size - at) ioFail("loadCheckpoint: '" + path + "' is truncated or corrupt");
        at += e.dataBytes;
        entries.push_back(std::move(e));
    }
    return entries;
}

namespace {
CheckpointLoadStats loadTensors(Model& model, const std::string& path, std::size_t chunkBytes, bool skipGemmWeights) {
    const auto t0 = std::chrono::steady_clock::now();
    const std::vector<CheckpointEntry> entries = indexCheckpoint(path);

    // names and shapes first: nothing is uploaded from a file that does not fit the model
    std::map<std::string, std::size_t> byName;
    for (std::size_t i = 0; i < model.parameterCount(); ++i) byName[model.parameterName(i)] = i;
    std::vector<std::size_t> target(entries.size());
    for (std::size_t i = 0; i < entries.size(); ++i) {
        auto it = byName.find(entries[i].name);
        if (it == byName.end()) ioFail("loadCheckpoint: the model has no parameter named '" + entries[i].name + "'");
        if (model.parameterShape(it->second) != entries[i].shape) {
            ioFail("loadCheckpoint: shape mismatch for '" + entries[i].name + "'");
        }
        target[i] = it->second;
    }

    // the work list: whole rows, never across tensors, at most about chunkBytes each
    if (chunkBytes == 0) chunkBytes = std::size_t(4) << 20;
    std::vector<Segment> segments;
    std::size_t largest = 0;
    CheckpointLoadStats stats;
    stats.tensors = entries.size();
    for (std::size_t i = 0; i < entries.size(); ++i) {
        const Model::RowView view = model.parameterRowView(target[i]);
        stats.fileBytes += entries[i].dataBytes;
        if (view.rows == 0 || view.rowElems == 0) continue;
        if (skipGemmWeights && model.parameterIsGemmWeight(target[i])) continue;   // their converted form is in place
        const std::size_t rowBytes = view.rowElems * sizeof(float);
        const std::size_t perChunk = std::max<std::size_t>(1, chunkBytes / rowBytes);
        for (std::size_t r = 0; r < view.neededRows; r += perChunk) {
            Segment s;
            s.param = target[i];
            s.firstRow = view.firstNeededRow + r;
            s.rows = std::min(perChunk, view.neededRows - r);
            s.offset = entries[i].dataOffset + static_cast<std::uint64_t>(s.firstRow) * rowBytes;
            s.bytes = s.rows * rowBytes;
            largest = std::max(largest, s.bytes);
            stats.readBytes += s.bytes;
            segments.push_back(s);
        }
    }
    if (segments.empty()) return stats;

    stats.uploadedBytes += streamSegments(path, segments, largest, [&](const Segment& seg, const void* host, cudaStream_t stream) {
        return model.uploadParameterRows(seg.param, seg.firstRow, seg.rows, static_cast<const float*>(host), stream);
    });
    model.invalidatePreparedWeights();
    stats.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return stats;
}

}  // namespace

CheckpointLoadStats loadCheckpoint(Model& model, const std::string& path, std::size_t chunkBytes) {
    return loadTensors(model, path, chunkBytes, false);
}

// ---- cache of converted weights beside the checkpoint ------------------------------------------------------
namespace {

constexpr char kCacheMagic[8] = {'B', 'F', 'B', '2', 'P', 'R', 'E', 'P'};
struct CacheHeader {
    char magic[8];
    std::uint32_t version;
    std::uint32_t pieces;
    std::uint64_t fingerprint;
    std::uint64_t sourceBytes;
    std::int64_t sourceMtimeNs;
};   // followed by `pieces` u64 sizes, then the pieces' bytes back to back

bool sourceIdentity(const std::string& path, std::uint64_t* bytes, std::int64_t* mtimeNs) {
    struct stat st {};
    if (::stat(path.c_str(), &st) != 0) return false;
    *bytes = static_cast<std::uint64_t>(st.st_size);
    *mtimeNs = static_cast<std::int64_t>(st.st_mtim.tv_sec) * 1000000000ll + st.st_mtim.tv_nsec;
    return true;
}

// The cache's data offset when the file is a valid cache of this checkpoint for this model, else 0.
std::uint64_t validCache(const std::string& cachePath, const CacheHeader& want, const std::vector<std::uint64_t>& sizes) {
    Fd file(cachePath);
    if (file.fd < 0) return 0;
    CacheHeader have{};
    if (readAt(file.fd, &have, sizeof(have), 0) != sizeof(have)) return 0;
    if (std::memcmp(have.magic, want.magic, sizeof(have.magic)) != 0 || have.version != want.version ||
        have.pieces != want.pieces || have.fingerprint != want.fingerprint || have.sourceBytes != want.sourceBytes ||
        have.sourceMtimeNs != want.sourceMtimeNs) {
        return 0;
    }
    std::vector<std::uint64_t> stored(sizes.size());
    const std::size_t tableBytes = sizes.size() * sizeof(std::uint64_t);
    if (readAt(file.fd, stored.data(), tableBytes, sizeof(have)) != tableBytes || stored != sizes) return 0;
    std::uint64_t total = sizeof(have) + tableBytes;
    for (std::uint64_t b : sizes) total += b;
    struct stat st {};
    if (::fstat(file.fd, &st) != 0 || static_cast<std::uint64_t>(st.st_size) != total) return 0;
    return sizeof(have) + tableBytes;
}

}  // namespace

CheckpointLoadStats loadCheckpointCached(Model& model, const std::string& path, std::size_t chunkBytes) {
    const auto t0 = std::chrono::steady_clock::now();
    const std::string tag = model.preparedWeightsTag();
    if (tag.empty()) return loadCheckpoint(model, path, chunkBytes);   // fp32 compute: nothing to cache
    const std::vector<CheckpointEntry> entries = indexCheckpoint(path);   // a missing or damaged checkpoint fails here, cache or not
    // A checkpoint may hold only some of the tensors (the loader keeps the model's own values for the rest, as the
    // reference does). The cache holds converted GEMM weights without saying where they came from, so it is written
    // and read only when every GEMM weight comes from the file: otherwise a weight the file lacks would be taken from
    // whichever model wrote the cache.
    {
        std::size_t covered = 0, wanted = 0;
        for (std::size_t i = 0; i < model.parameterCount(); ++i) {
            if (!model.parameterIsGemmWeight(i)) continue;
            ++wanted;
            for (const CheckpointEntry& e : entries) {
                if (e.name == model.parameterName(i)) {
                    ++covered;
                    break;
                }
            }
        }
        if (covered != wanted) return loadCheckpoint(model, path, chunkBytes);
    }
    if (chunkBytes == 0) chunkBytes = std::size_t(4) << 20;
    const std::string cachePath = path + ".bfb200cache." + tag;
    CacheHeader want{};
    std::memcpy(want.magic, kCacheMagic, sizeof(kCacheMagic));
    want.version = 1;
    want.fingerprint = model.structureFingerprint();
    if (!sourceIdentity(path, &want.sourceBytes, &want.sourceMtimeNs)) ioFail("loadCheckpoint: cannot stat '" + path + "'");

    std::vector<Model::PreparedPiece> pieces = model.preparedWeightPieces(true);
    std::vector<std::uint64_t> sizes;
    for (const Model::PreparedPiece& p : pieces) sizes.push_back(p.bytes);
    want.pieces = static_cast<std::uint32_t>(pieces.size());

    const std::uint64_t dataAt = validCache(cachePath, want, sizes);
    if (dataAt != 0) {
        std::vector<Segment> segments;
        std::size_t largest = 0;
        std::uint64_t at = dataAt, cacheBytes = 0;
        for (const Model::PreparedPiece& p : pieces) {
            for (std::size_t done = 0; done < p.bytes; done += chunkBytes) {
                Segment s;
                s.offset = at + done;
                s.bytes = std::min(chunkBytes, p.bytes - done);
                s.deviceDst = static_cast<char*>(p.data) + done;
                largest = std::max(largest, s.bytes);
                segments.push_back(s);
            }
            at += p.bytes;
            cacheBytes += p.bytes;
        }
        const std::size_t sent = streamSegments(cachePath, segments, largest, [](const Segment& seg, const void* host, cudaStream_t stream) {
            BFB_CUDA(cudaMemcpyAsync(seg.deviceDst, host, seg.bytes, cudaMemcpyHostToDevice, stream));
            return seg.bytes;
        });
        model.adoptPreparedWeights();
        CheckpointLoadStats stats = loadTensors(model, path, chunkBytes, true);   // tables, biases
        stats.cacheHit = true;
        stats.cacheBytes = cacheBytes;
        stats.readBytes += cacheBytes;
        stats.uploadedBytes += sent;
        stats.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        return stats;
    }

    // miss: the ordinary load, one conversion, and the cache for next time (written beside, renamed into place)
    CheckpointLoadStats stats = loadCheckpoint(model, path, chunkBytes);
    pieces = model.preparedWeightPieces(false);
    const std::string tmpPath = cachePath + ".tmp" + std::to_string(static_cast<long long>(::getpid()));
    {
        std::ofstream out(tmpPath, std::ios::binary | std::ios::trunc);
        if (!out) return stats;   // a read-only directory: no cache, no error
        out.write(reinterpret_cast<const char*>(&want), sizeof(want));
        out.write(reinterpret_cast<const char*>(sizes.data()), static_cast<std::streamsize>(sizes.size() * sizeof(std::uint64_t)));
        std::vector<char> host(std::min<std::size_t>(std::size_t(64) << 20, std::max<std::size_t>(chunkBytes, 1)));
        for (const Model::PreparedPiece& p : pieces) {
            for (std::size_t done = 0; done < p.bytes; done += host.size()) {
                const std::size_t n = std::min(host.size(), p.bytes - done);
                BFB_CUDA(cudaMemcpy(host.data(), static_cast<const char*>(p.data) + done, n, cudaMemcpyDeviceToHost));
                out.write(host.data(), static_cast<std::streamsize>(n));
            }
            stats.cacheBytes += p.bytes;
        }
        if (!out) {
            out.close();
            ::unlink(tmpPath.c_str());
            stats.cacheBytes = 0;
            return stats;
        }
    }
    if (::rename(tmpPath.c_str(), cachePath.c_str()) != 0) {
        ::unlink(tmpPath.c_str());
        stats.cacheBytes = 0;
    }
    stats.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return stats;
}

void saveCheckpoint(Model& model, const std::string& path) {
    std::vector<Parameter*> params = model.parameters();
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    if (!out) ioFail("saveCheckpoint: cannot write '" + path + "'");
    out.write(kMagic, sizeof(kMagic));
    auto u32 = [&](std::uint32_t v) { out.write(reinterpret_cast<const char*>(&v), sizeof(v)); };
    auto u64 = [&](std::uint64_t v) { out.write(reinterpret_cast<const char*>(&v), sizeof(v)); };
    u32(static_cast<std::uint32_t>(params.size()));
    std::vector<float> host;
    for (std::size_t i = 0; i < params.size(); ++i) {
        const Parameter& p = *params[i];
        u32(static_cast<std::uint32_t>(p.name.size()));
        out.write(p.name.data(), static_cast<std::streamsize>(p.name.size()));
        u32(static_cast<std::uint32_t>(p.fullShape.size()));
        std::size_t count = 1;
        for (std::size_t d : p.fullShape) {
            u64(static_cast<std::uint64_t>(d));
            count *= d;
        }
        host.resize(count);
        model.getParameter(i, host.data());
        out.write(reinterpret_cast<const char*>(host.data()), static_cast<std::streamsize>(count * sizeof(float)));
    }
    if (!out) ioFail("saveCheckpoint: write to '" + path + "' failed");
}

}  // namespace bfb200
