// Host runtime, part 3: parallel file reader for checkpoint loading. A checkpoint shard is read
// as a list of (file offset, byte count, destination) ranges by a pool of threads with pread();
// destinations are caller-owned (pinned host staging the loader then copies to the device with one
// async H2D per tensor), so reading the next tensors overlaps the copies of the previous ones.
// O_DIRECT is used when asked for and the range is aligned, with a buffered read of the ragged
// head and tail; it keeps a 100 GB checkpoint from evicting the page cache.
// Role of the reference's crates/model-weights/src/fast_weights (O_DIRECT + pipelined H2D).
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int64_t kAlign = 4096;
constexpr int64_t kChunk = 8 << 20;       // work unit: large ranges are split so threads balance

struct Piece { int64_t off, len; uint8_t* dst; };

int64_t pread_all(int fd, uint8_t* dst, int64_t len, int64_t off) {
  int64_t done = 0;
  while (done < len) {
    ssize_t r = ::pread(fd, dst + done, static_cast<size_t>(len - done), off + done);
    if (r < 0) {
      if (errno == EINTR) continue;
      return -errno;
    }
    if (r == 0) return -EIO;            // short file
    done += r;
  }
  return done;
}

}  // namespace

extern "C" {

// Reads n ranges of `path`. Returns total bytes read, or a negative errno.
int64_t mrt_read_ranges(const char* path, int32_t n, const int64_t* offsets, const int64_t* sizes,
                        uint8_t* const* dsts, int32_t threads, int32_t direct) {
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -errno;
  int dfd = -1;
  if (direct) dfd = ::open(path, O_RDONLY | O_DIRECT);      // may fail (tmpfs): fall back to buffered
  std::vector<Piece> pieces;
  for (int32_t i = 0; i < n; ++i)
    for (int64_t o = 0; o < sizes[i]; o += kChunk)
      pieces.push_back({offsets[i] + o, sizes[i] - o < kChunk ? sizes[i] - o : kChunk, dsts[i] + o});
  std::atomic<size_t> next{0};
  std::atomic<int64_t> total{0}, err{0};
  auto work = [&]() {
    void* bounce = nullptr;
    if (dfd >= 0 && ::posix_memalign(&bounce, kAlign, kChunk + 2 * kAlign) != 0) bounce = nullptr;
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= pieces.size() || err.load() != 0) break;
      const Piece& p = pieces[i];
      int64_t r;
      if (dfd >= 0 && bounce) {
        // aligned window covering the piece, read into the bounce buffer, then copied out
        int64_t a0 = p.off / kAlign * kAlign;
        int64_t a1 = (p.off + p.len + kAlign - 1) / kAlign * kAlign;
        int64_t got = 0;
        while (got < a1 - a0) {
          ssize_t k = ::pread(dfd, static_cast<uint8_t*>(bounce) + got, static_cast<size_t>(a1 - a0 - got), a0 + got);
          if (k < 0 && errno == EINTR) continue;
          if (k <= 0) break;              // end of file inside the last aligned block is fine
          got += k;
        }
        if (got >= p.off - a0 + p.len) {
          std::memcpy(p.dst, static_cast<uint8_t*>(bounce) + (p.off - a0), static_cast<size_t>(p.len));
          r = p.len;
        } else {
          r = pread_all(fd, p.dst, p.len, p.off);
        }
      } else {
        r = pread_all(fd, p.dst, p.len, p.off);
      }
      if (r < 0) { err.store(r); break; }
      total.fetch_add(r);
    }
    std::free(bounce);
  };
  int nt = threads < 1 ? 1 : (threads > 64 ? 64 : threads);
  if (static_cast<size_t>(nt) > pieces.size()) nt = pieces.empty() ? 1 : static_cast<int>(pieces.size());
  std::vector<std::thread> pool;
  for (int t = 1; t < nt; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  ::close(fd);
  if (dfd >= 0) ::close(dfd);
  return err.load() != 0 ? err.load() : total.load();
}

}  // extern "C"
