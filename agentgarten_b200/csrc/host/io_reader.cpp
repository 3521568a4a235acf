// Parallel positional file reader: the host half of weight loading.
//
// A checkpoint tensor file is read as many independent byte ranges.  Each range is cut
// into chunks; a pool of threads takes chunks from one atomic counter and issues pread()
// straight into the caller's (usually pinned) memory, so a network or striped filesystem
// sees many requests in flight and the copy engine can start on a slab as soon as the
// call returns.  The interpreter lock is released for the whole call.
//
// Python surface (module agentgarten_b200._io):
//   read_ranges(path, ranges, threads=16, chunk=64<<20) -> bytes read
//     ranges: sequence of (file_offset, size, destination_address)
//   file_size(path) -> int
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <stdexcept>
#include <string>
#include <sys/stat.h>
#include <thread>
#include <tuple>
#include <unistd.h>
#include <vector>

namespace py = pybind11;

namespace {

struct Chunk {
    int64_t offset;
    int64_t size;
    char* destination;
};

struct FileHandle {
    int fd;
    explicit FileHandle(const std::string& path) : fd(::open(path.c_str(), O_RDONLY | O_CLOEXEC)) {
        if (fd < 0) throw std::runtime_error("cannot open " + path + ": " + std::strerror(errno));
    }
    ~FileHandle() { if (fd >= 0) ::close(fd); }
    FileHandle(const FileHandle&) = delete;
    FileHandle& operator=(const FileHandle&) = delete;
};

int64_t read_ranges(const std::string& path,
                    const std::vector<std::tuple<int64_t, int64_t, uint64_t>>& ranges,
                    int threads, int64_t chunk) {
    if (chunk <= 0) throw std::invalid_argument("chunk must be positive");
    std::vector<Chunk> work;
    int64_t total = 0;
    for (const auto& [offset, size, address] : ranges) {
        if (offset < 0 || size < 0) throw std::invalid_argument("negative offset or size");
        if (size > 0 && address == 0) throw std::invalid_argument("null destination");
        for (int64_t done = 0; done < size; done += chunk) {
            const int64_t piece = std::min(chunk, size - done);
            work.push_back({offset + done, piece, reinterpret_cast<char*>(address) + done});
        }
        total += size;
    }
    if (work.empty()) return 0;
    FileHandle file(path);
    struct stat info {};
    if (::fstat(file.fd, &info) != 0) throw std::runtime_error("fstat failed on " + path);
    for (const auto& c : work)
        if (c.offset + c.size > info.st_size)
            throw std::runtime_error("range past the end of " + path + " (truncated file?)");

    std::atomic<size_t> next{0};
    std::atomic<bool> failed{false};
    std::mutex error_lock;
    std::string error;
    auto worker = [&]() {
        while (!failed.load(std::memory_order_relaxed)) {
            const size_t index = next.fetch_add(1, std::memory_order_relaxed);
            if (index >= work.size()) return;
            const Chunk& c = work[index];
            int64_t done = 0;
            while (done < c.size) {
                const ssize_t got = ::pread(file.fd, c.destination + done, size_t(c.size - done), c.offset + done);
                if (got > 0) { done += got; continue; }
                if (got < 0 && errno == EINTR) continue;
                std::lock_guard<std::mutex> hold(error_lock);
                error = got == 0 ? "unexpected end of file" : std::strerror(errno);
                failed.store(true);
                return;
            }
        }
    };
    {
        py::gil_scoped_release release;
        const int count = std::max(1, std::min<int>(threads, int(work.size())));
        std::vector<std::thread> pool;
        pool.reserve(size_t(count));
        for (int i = 0; i + 1 < count; ++i) pool.emplace_back(worker);
        worker();  // the calling thread takes its share
        for (auto& t : pool) t.join();
    }
    if (failed.load()) throw std::runtime_error("read of " + path + " failed: " + error);
    return total;
}

int64_t file_size(const std::string& path) {
    struct stat info {};
    if (::stat(path.c_str(), &info) != 0) throw std::runtime_error("cannot stat " + path);
    return int64_t(info.st_size);
}

}  // namespace

PYBIND11_MODULE(_io, m) {
    m.doc() = "parallel positional reads into caller-owned memory";
    m.def("read_ranges", &read_ranges, py::arg("path"), py::arg("ranges"), py::arg("threads") = 16,
          py::arg("chunk") = int64_t(64) << 20);
    m.def("file_size", &file_size, py::arg("path"));
}
