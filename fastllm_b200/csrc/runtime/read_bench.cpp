// Storage read-throughput probe for weight files (the figure that bounds cold model loads and the "disk" expert placement).
// Worker threads take fixed-size extents from ONE shared cursor that runs over all files back to back (and wraps), so the
// load spreads over files and offsets whatever the thread count; reads go through pread into page-aligned buffers,
// optionally with O_DIRECT to bypass the page cache.  Counterpart of the reference's tools/ssd_read_bench.cpp (which gives
// every thread its own file sequence).
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

extern "C" int fbio_read_bench(const char* const* paths, int n_paths, int threads, double seconds, long long block_bytes, int direct,
                               unsigned long long* out_bytes, unsigned long long* out_reads, double* out_elapsed) {
  if (n_paths <= 0 || threads <= 0 || block_bytes <= 0) return -1;
  block_bytes = (block_bytes + 4095) / 4096 * 4096;
  struct File { std::string path; long long size; long long first_extent; };
  std::vector<File> files;
  long long extents = 0;
  for (int i = 0; i < n_paths; ++i) {
    struct stat st;
    if (stat(paths[i], &st) != 0 || !S_ISREG(st.st_mode) || st.st_size <= 0) continue;
    files.push_back({paths[i], (long long)st.st_size, extents});
    extents += (st.st_size + block_bytes - 1) / block_bytes;
  }
  if (files.empty()) return -2;
  std::atomic<unsigned long long> bytes{0}, reads{0}, cursor{0};
  std::atomic<int> errors{0};
  std::atomic<bool> go{false};
  std::vector<std::thread> pool;
  const auto run_for = std::chrono::duration<double>(seconds);
  std::chrono::steady_clock::time_point t_begin;
  for (int t = 0; t < threads; ++t) {
    pool.emplace_back([&]() {
      void* buf = nullptr;
      if (posix_memalign(&buf, 4096, (size_t)block_bytes) != 0) { errors++; return; }
      std::vector<int> fds(files.size(), -1);
      while (!go.load(std::memory_order_acquire)) std::this_thread::yield();
      const auto deadline = t_begin + std::chrono::duration_cast<std::chrono::steady_clock::duration>(run_for);
      unsigned long long local_bytes = 0, local_reads = 0;
      while (std::chrono::steady_clock::now() < deadline) {
        const long long ext = (long long)(cursor.fetch_add(1, std::memory_order_relaxed) % (unsigned long long)extents);
        size_t fi = 0;                                  // file that holds this extent (few files: linear scan)
        while (fi + 1 < files.size() && files[fi + 1].first_extent <= ext) ++fi;
        if (fds[fi] < 0) {
          int flags = O_RDONLY;
#ifdef O_DIRECT
          if (direct) flags |= O_DIRECT;
#endif
          fds[fi] = open(files[fi].path.c_str(), flags);
          if (fds[fi] < 0) { errors++; break; }
        }
        const long long off = (ext - files[fi].first_extent) * block_bytes;
        const ssize_t got = pread(fds[fi], buf, (size_t)block_bytes, (off_t)off);
        if (got < 0) { errors++; break; }
        local_bytes += (unsigned long long)got;
        ++local_reads;
      }
      for (int fd : fds) if (fd >= 0) close(fd);
      free(buf);
      bytes += local_bytes;
      reads += local_reads;
    });
  }
  t_begin = std::chrono::steady_clock::now();
  go.store(true, std::memory_order_release);
  for (auto& th : pool) th.join();
  const double elapsed = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_begin).count();
  if (out_bytes) *out_bytes = bytes.load();
  if (out_reads) *out_reads = reads.load();
  if (out_elapsed) *out_elapsed = elapsed;
  return errors.load() ? -3 : 0;
}
