// Host-side runtime pieces that are worth doing natively: the sequence packer that runs between
// rollout and training, parallel positional reads for checkpoint / safetensors loading, and an
// asynchronous file writer for checkpoints. Plain C++17 + pthreads, C ABI, no CUDA calls.
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

#include <errno.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

// ------------------------------------------------------------------------------------------------
// First-fit-decreasing packing of n items into `pack_size` bins, each bounded by `budget` tokens and
// `max_segments` items. assign[i] = bin of item i, or -1 when it fits nowhere. Ties keep input order.
// ------------------------------------------------------------------------------------------------
extern "C" int tx_ffd_pack(const int* lengths, int n, int pack_size, long long budget, int max_segments,
                           int* assign) {
  if (n < 0 || pack_size <= 0 || !assign || (n > 0 && !lengths)) return 1;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lengths[a] > lengths[b]; });
  std::vector<long long> load(pack_size, 0);
  std::vector<int> count(pack_size, 0);
  int first_open = 0;   // bins before this one are full in tokens or segments for every remaining item
  for (int idx : order) {
    assign[idx] = -1;
    const long long len = lengths[idx];
    for (int b = first_open; b < pack_size; ++b) {
      if (load[b] + len <= budget && count[b] < max_segments) {
        assign[idx] = b;
        load[b] += len;
        ++count[b];
        break;
      }
    }
    while (first_open < pack_size && (count[first_open] >= max_segments || load[first_open] >= budget)) ++first_open;
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Parallel positional read: nbytes from `path` at `offset` into dst with up to `threads` pread loops.
// Returns 0, or an errno value.
// ------------------------------------------------------------------------------------------------
extern "C" int tx_pread_parallel(const char* path, long long offset, long long nbytes, void* dst, int threads) {
  if (!path || !dst || offset < 0 || nbytes < 0) return EINVAL;
  if (nbytes == 0) return 0;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return errno;
  const long long min_chunk = 8LL << 20;
  int nt = static_cast<int>(std::min<long long>(std::max(threads, 1), (nbytes + min_chunk - 1) / min_chunk));
  std::atomic<int> err{0};
  auto work = [&](long long lo, long long hi) {
    long long pos = lo;
    while (pos < hi && err.load() == 0) {
      const ssize_t got = pread(fd, static_cast<char*>(dst) + pos, static_cast<size_t>(std::min<long long>(hi - pos, 64LL << 20)),
                                offset + pos);
      if (got < 0) {
        if (errno == EINTR) continue;
        err.store(errno);
        return;
      }
      if (got == 0) {
        err.store(EIO);   // file shorter than promised
        return;
      }
      pos += got;
    }
  };
  std::vector<std::thread> pool;
  const long long per = (nbytes + nt - 1) / nt;
  for (int t = 1; t < nt; ++t) pool.emplace_back(work, t * per, std::min(nbytes, (t + 1) * per));
  work(0, std::min(nbytes, per));
  for (auto& th : pool) th.join();
  close(fd);
  return err.load();
}

// ------------------------------------------------------------------------------------------------
// Asynchronous writer: submit(path, bytes) copies nothing - the caller keeps the buffer alive until
// wait() returns - writes to "<path>.tmp.<id>", optionally fsyncs, then renames into place.
// ------------------------------------------------------------------------------------------------
namespace {
struct WriteJob {
  std::string path;
  const void* data;
  long long nbytes;
  int do_fsync;
};

struct Writer {
  std::mutex mu;
  std::condition_variable cv_work, cv_idle;
  std::deque<WriteJob> queue;
  std::vector<std::thread> threads;
  int in_flight = 0;
  int errors = 0;
  int first_errno = 0;
  bool stop = false;
  std::atomic<unsigned long long> seq{0};

  void run() {
    for (;;) {
      WriteJob job;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv_work.wait(lk, [&] { return stop || !queue.empty(); });
        if (queue.empty()) return;
        job = std::move(queue.front());
        queue.pop_front();
      }
      const int rc = write_one(job);
      {
        std::lock_guard<std::mutex> lk(mu);
        if (rc != 0) {
          ++errors;
          if (first_errno == 0) first_errno = rc;
        }
        --in_flight;
        if (in_flight == 0) cv_idle.notify_all();
      }
    }
  }

  int write_one(const WriteJob& job) {
    const std::string tmp = job.path + ".tmp." + std::to_string(seq.fetch_add(1));
    const int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) return errno;
    long long pos = 0;
    int rc = 0;
    while (pos < job.nbytes) {
      const ssize_t put = write(fd, static_cast<const char*>(job.data) + pos,
                                static_cast<size_t>(std::min<long long>(job.nbytes - pos, 64LL << 20)));
      if (put < 0) {
        if (errno == EINTR) continue;
        rc = errno;
        break;
      }
      pos += put;
    }
    if (rc == 0 && job.do_fsync && fsync(fd) != 0) rc = errno;
    if (close(fd) != 0 && rc == 0) rc = errno;
    if (rc == 0 && rename(tmp.c_str(), job.path.c_str()) != 0) rc = errno;
    if (rc != 0) unlink(tmp.c_str());
    return rc;
  }
};
}  // namespace

extern "C" void* tx_writer_create(int threads) {
  auto* w = new Writer();
  const int n = std::max(1, std::min(threads, 64));
  for (int i = 0; i < n; ++i) w->threads.emplace_back([w] { w->run(); });
  return w;
}

extern "C" int tx_writer_submit(void* handle, const char* path, const void* data, long long nbytes, int do_fsync) {
  auto* w = static_cast<Writer*>(handle);
  if (!w || !path || nbytes < 0 || (nbytes > 0 && !data)) return EINVAL;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    if (w->stop) return EINVAL;
    w->queue.push_back(WriteJob{path, data, nbytes, do_fsync});
    ++w->in_flight;
  }
  w->cv_work.notify_one();
  return 0;
}

// Blocks until every submitted write has finished; returns the number of failed writes since the last
// call and stores the first errno in *first_errno (may be null).
extern "C" int tx_writer_wait(void* handle, int* first_errno) {
  auto* w = static_cast<Writer*>(handle);
  if (!w) return -1;
  std::unique_lock<std::mutex> lk(w->mu);
  w->cv_idle.wait(lk, [&] { return w->in_flight == 0; });
  const int e = w->errors;
  if (first_errno) *first_errno = w->first_errno;
  w->errors = 0;
  w->first_errno = 0;
  return e;
}

extern "C" void tx_writer_destroy(void* handle) {
  auto* w = static_cast<Writer*>(handle);
  if (!w) return;
  {
    std::lock_guard<std::mutex> lk(w->mu);
    w->stop = true;
  }
  w->cv_work.notify_all();
  for (auto& t : w->threads) t.join();
  delete w;
}
