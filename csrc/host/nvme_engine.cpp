// Asynchronous file I/O engine for the NVMe tier.
//
// A handle owns `threads` workers.  Every submitted transfer is cut into
// per-worker byte ranges; each worker drives its range through its own
// io_uring (raw syscalls - no liburing on the target image) keeping up to
// `queue_depth` block-sized requests in flight, falls back to Linux native AIO
// syscalls, and finally to pread/pwrite.  Files are opened O_DIRECT when the
// file system accepts it and kept in an fd cache until the handle dies.
// Errors are returned as negative errno values, never asserted.  A fault
// injector (tests only) makes the next N block transfers fail or come up short.
//
// Capability parity: flextrain/ops/csrc/aio/common/deepspeed_aio_common.cpp:71-341,
// flextrain/ops/csrc/aio/py_lib/deepspeed_py_io_handle.cpp:37-355,
// deepspeed_aio_thread.cpp:24-51, deepspeed_py_aio.cpp:39-123.
#include <errno.h>
#include <fcntl.h>
#include <linux/aio_abi.h>
#include <linux/io_uring.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <sys/uio.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

enum EngineKind : int { kAuto = 0, kUring = 1, kAio = 2, kPsync = 3 };

// ----------------------------------------------------------- raw io_uring
struct Uring {
  int fd = -1;
  unsigned entries = 0;
  void* sq_ptr = nullptr;
  size_t sq_len = 0;
  void* cq_ptr = nullptr;
  size_t cq_len = 0;
  io_uring_sqe* sqes = nullptr;
  size_t sqes_len = 0;
  unsigned *sq_head, *sq_tail, *sq_mask, *sq_array;
  unsigned *cq_head, *cq_tail, *cq_mask;
  io_uring_cqe* cqes = nullptr;

  bool init(unsigned depth) {
    io_uring_params p;
    std::memset(&p, 0, sizeof(p));
    fd = (int)syscall(__NR_io_uring_setup, depth, &p);
    if (fd < 0) return false;
    entries = p.sq_entries;
    sq_len = p.sq_off.array + p.sq_entries * sizeof(unsigned);
    cq_len = p.cq_off.cqes + p.cq_entries * sizeof(io_uring_cqe);
    bool single = p.features & IORING_FEAT_SINGLE_MMAP;
    if (single) sq_len = cq_len = sq_len > cq_len ? sq_len : cq_len;
    sq_ptr = mmap(nullptr, sq_len, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd,
                  IORING_OFF_SQ_RING);
    if (sq_ptr == MAP_FAILED) { sq_ptr = nullptr; destroy(); return false; }
    if (single) {
      cq_ptr = sq_ptr;
    } else {
      cq_ptr = mmap(nullptr, cq_len, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd,
                    IORING_OFF_CQ_RING);
      if (cq_ptr == MAP_FAILED) { cq_ptr = nullptr; destroy(); return false; }
    }
    sqes_len = p.sq_entries * sizeof(io_uring_sqe);
    sqes = (io_uring_sqe*)mmap(nullptr, sqes_len, PROT_READ | PROT_WRITE,
                               MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQES);
    if (sqes == MAP_FAILED) { sqes = nullptr; destroy(); return false; }
    char* sq = (char*)sq_ptr;
    sq_head = (unsigned*)(sq + p.sq_off.head);
    sq_tail = (unsigned*)(sq + p.sq_off.tail);
    sq_mask = (unsigned*)(sq + p.sq_off.ring_mask);
    sq_array = (unsigned*)(sq + p.sq_off.array);
    char* cq = (char*)cq_ptr;
    cq_head = (unsigned*)(cq + p.cq_off.head);
    cq_tail = (unsigned*)(cq + p.cq_off.tail);
    cq_mask = (unsigned*)(cq + p.cq_off.ring_mask);
    cqes = (io_uring_cqe*)(cq + p.cq_off.cqes);
    return true;
  }

  void destroy() {
    if (sqes) munmap(sqes, sqes_len);
    if (cq_ptr && cq_ptr != sq_ptr) munmap(cq_ptr, cq_len);
    if (sq_ptr) munmap(sq_ptr, sq_len);
    if (fd >= 0) close(fd);
    sqes = nullptr; cq_ptr = sq_ptr = nullptr; fd = -1;
  }

  // queue one read/write; caller guarantees in-flight < entries.  `fixed` >= 0 names a
  // registered buffer that contains [buf, buf + len): the kernel then skips pinning the
  // pages for this request.
  void push(bool write, int file, void* buf, unsigned len, uint64_t off, uint64_t tag, int fixed = -1) {
    unsigned tail = *sq_tail;
    unsigned idx = tail & *sq_mask;
    io_uring_sqe* e = &sqes[idx];
    std::memset(e, 0, sizeof(*e));
    if (fixed >= 0) {
      e->opcode = write ? IORING_OP_WRITE_FIXED : IORING_OP_READ_FIXED;
      e->buf_index = (uint16_t)fixed;
    } else {
      e->opcode = write ? IORING_OP_WRITE : IORING_OP_READ;
    }
    e->fd = file;
    e->addr = (uint64_t)buf;
    e->len = len;
    e->off = off;
    e->user_data = tag;
    sq_array[idx] = idx;
    __atomic_store_n(sq_tail, tail + 1, __ATOMIC_RELEASE);
  }

  int enter(unsigned to_submit, unsigned min_complete) {
    for (;;) {
      int r = (int)syscall(__NR_io_uring_enter, fd, to_submit, min_complete,
                           min_complete ? IORING_ENTER_GETEVENTS : 0, nullptr, 0);
      if (r < 0 && errno == EINTR) continue;
      return r < 0 ? -errno : r;
    }
  }

  // (Re)register a set of buffers; n == 0 just drops the current set.  0 or -errno.
  int register_buffers(const iovec* iov, unsigned n) {
    syscall(__NR_io_uring_register, fd, IORING_UNREGISTER_BUFFERS, nullptr, 0);   // fine if none
    if (n == 0) return 0;
    long r = syscall(__NR_io_uring_register, fd, IORING_REGISTER_BUFFERS, iov, n);
    return r < 0 ? -errno : 0;
  }

  bool pop(io_uring_cqe* out) {
    unsigned head = *cq_head;
    if (head == __atomic_load_n(cq_tail, __ATOMIC_ACQUIRE)) return false;
    *out = cqes[head & *cq_mask];
    __atomic_store_n(cq_head, head + 1, __ATOMIC_RELEASE);
    return true;
  }
};

// ---------------------------------------------------------------- engine
struct SubOp {
  int64_t op_id;
  bool write;
  int fd;
  char* buf;
  int64_t nbytes;
  int64_t file_off;
};

struct OpState {
  std::atomic<int> remaining{0};
  std::atomic<int> error{0};
};

struct Engine;

struct Worker {
  Engine* eng = nullptr;
  std::thread th;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<SubOp> q;
  bool stop = false;
  Uring ring;
  bool ring_ok = false;
  std::atomic<bool> ring_registered{false};  // this worker's ring holds Engine::reg
  aio_context_t aio_ctx = 0;
  bool aio_ok = false;
};

struct Engine {
  int64_t block_size;
  int queue_depth;
  int n_threads;
  int kind;        // resolved engine
  bool want_direct;
  std::vector<std::unique_ptr<Worker>> workers;

  std::mutex fd_mu;
  std::map<std::string, int> fds;            // key: path + mode
  std::map<std::string, bool> fd_is_direct;

  std::mutex op_mu;
  std::condition_variable op_cv;
  std::map<int64_t, std::shared_ptr<OpState>> ops;
  int64_t next_op = 1;
  int64_t completed_since_wait = 0;
  int first_error = 0;

  std::atomic<int> fault_kind{0};            // 0 none, 1 EIO, 2 short transfer
  std::atomic<int> fault_countdown{0};
  std::atomic<int64_t> bytes_read{0}, bytes_written{0};

  // registered (page-locked) buffers of the io_uring workers, split into <= 1 GiB pieces
  std::mutex reg_mu;
  std::vector<iovec> reg;                    // index == buf_index in every worker's ring
  std::atomic<int64_t> fixed_ops{0};
};

// index of the registered piece that contains [p, p + len), or -1
int find_registered(Engine* e, const char* p, int64_t len) {
  std::lock_guard<std::mutex> lk(e->reg_mu);
  for (size_t i = 0; i < e->reg.size(); ++i) {
    const char* b = (const char*)e->reg[i].iov_base;
    if (p >= b && p + len <= b + e->reg[i].iov_len) return (int)i;
  }
  return -1;
}

int consume_fault(Engine* e) {
  int k = e->fault_kind.load();
  if (!k) return 0;
  int c = e->fault_countdown.fetch_sub(1);
  if (c <= 0) { e->fault_countdown.store(0); e->fault_kind.store(0); return 0; }
  return k;
}

void finish_subop(Engine* e, const SubOp& s, int err) {
  std::shared_ptr<OpState> st;
  {
    std::lock_guard<std::mutex> lk(e->op_mu);
    auto it = e->ops.find(s.op_id);
    if (it == e->ops.end()) return;
    st = it->second;
  }
  if (err) { int z = 0; st->error.compare_exchange_strong(z, err); }
  if (st->remaining.fetch_sub(1) == 1) {
    std::lock_guard<std::mutex> lk(e->op_mu);
    e->completed_since_wait += 1;
    if (st->error.load() && !e->first_error) e->first_error = st->error.load();
    e->op_cv.notify_all();
  }
}

int run_psync(Engine* e, const SubOp& s) {
  int64_t done = 0;
  while (done < s.nbytes) {
    int64_t len = s.nbytes - done < e->block_size ? s.nbytes - done : e->block_size;
    int f = consume_fault(e);
    if (f == 1) return -EIO;
    ssize_t r = s.write ? pwrite(s.fd, s.buf + done, (size_t)len, s.file_off + done)
                        : pread(s.fd, s.buf + done, (size_t)len, s.file_off + done);
    if (f == 2 && r > 1) r = r / 2;   // pretend the kernel came up short
    if (r < 0) { if (errno == EINTR) continue; return -errno; }
    if (r == 0) return -ENODATA;      // read past end of file
    if (f == 2) return -EIO;          // a short transfer that is not retried
    done += r;
  }
  return 0;
}

int run_uring(Engine* e, Worker* w, const SubOp& s) {
  int64_t issued = 0, completed_bytes = 0;
  int inflight = 0, err = 0;
  const int depth = (int)w->ring.entries < e->queue_depth ? (int)w->ring.entries : e->queue_depth;
  while (completed_bytes < s.nbytes && !err) {
    unsigned batch = 0;
    while (issued < s.nbytes && inflight < depth) {
      int64_t len = s.nbytes - issued < e->block_size ? s.nbytes - issued : e->block_size;
      int f = consume_fault(e);
      if (f) { err = -EIO; break; }
      const int fixed = w->ring_registered ? find_registered(e, s.buf + issued, len) : -1;
      if (fixed >= 0) e->fixed_ops.fetch_add(1);
      w->ring.push(s.write, s.fd, s.buf + issued, (unsigned)len, (uint64_t)(s.file_off + issued),
                   (uint64_t)len, fixed);
      issued += len; ++inflight; ++batch;
    }
    if (inflight == 0) break;
    int r = w->ring.enter(batch, 1);
    if (r < 0) { err = r; break; }
    io_uring_cqe c;
    while (w->ring.pop(&c)) {
      --inflight;
      if (c.res < 0) { if (!err) err = c.res; }
      else if ((uint64_t)c.res != c.user_data) { if (!err) err = c.res == 0 ? -ENODATA : -EIO; }
      else completed_bytes += c.res;
    }
  }
  // drain whatever is still in flight so the buffers are safe to reuse
  int spins = 0;
  while (inflight > 0 && spins < 1000000) {
    int r = w->ring.enter(0, 1);
    if (r < 0) break;
    io_uring_cqe c;
    while (w->ring.pop(&c)) --inflight;
    ++spins;
  }
  return err;
}

int run_aio(Engine* e, Worker* w, const SubOp& s) {
  const int depth = e->queue_depth;
  std::vector<iocb> cbs(depth);
  std::vector<iocb*> ptrs(depth);
  std::vector<io_event> events(depth);
  int64_t issued = 0, completed_bytes = 0;
  int inflight = 0, err = 0;
  std::vector<int> free_slots;
  for (int i = depth - 1; i >= 0; --i) free_slots.push_back(i);
  while (completed_bytes < s.nbytes && !err) {
    int batch = 0;
    while (issued < s.nbytes && !free_slots.empty()) {
      int64_t len = s.nbytes - issued < e->block_size ? s.nbytes - issued : e->block_size;
      if (consume_fault(e)) { err = -EIO; break; }
      int slot = free_slots.back(); free_slots.pop_back();
      iocb* cb = &cbs[slot];
      std::memset(cb, 0, sizeof(*cb));
      cb->aio_fildes = s.fd;
      cb->aio_lio_opcode = s.write ? IOCB_CMD_PWRITE : IOCB_CMD_PREAD;
      cb->aio_buf = (uint64_t)(s.buf + issued);
      cb->aio_nbytes = (uint64_t)len;
      cb->aio_offset = s.file_off + issued;
      cb->aio_data = ((uint64_t)slot << 40) | (uint64_t)len;
      ptrs[batch++] = cb;
      issued += len;
    }
    if (batch) {
      int done = 0;
      while (done < batch) {
        long r = syscall(__NR_io_submit, w->aio_ctx, (long)(batch - done), ptrs.data() + done);
        if (r < 0) { if (errno == EINTR || errno == EAGAIN) continue; err = -errno; break; }
        done += (int)r;
      }
      inflight += done;
      if (err) break;
    }
    if (inflight == 0) break;
    long n = syscall(__NR_io_getevents, w->aio_ctx, 1L, (long)depth, events.data(), nullptr);
    if (n < 0) { if (errno == EINTR) continue; err = -errno; break; }
    for (long i = 0; i < n; ++i) {
      --inflight;
      int slot = (int)(events[i].data >> 40);
      int64_t want = (int64_t)(events[i].data & ((1ull << 40) - 1));
      free_slots.push_back(slot);
      if ((int64_t)events[i].res < 0) { if (!err) err = (int)events[i].res; }
      else if ((int64_t)events[i].res != want) { if (!err) err = -EIO; }
      else completed_bytes += want;
    }
  }
  while (inflight > 0) {
    long n = syscall(__NR_io_getevents, w->aio_ctx, 1L, (long)depth, events.data(), nullptr);
    if (n <= 0) break;
    inflight -= (int)n;
  }
  return err;
}

void worker_loop(Worker* w) {
  Engine* e = w->eng;
  for (;;) {
    SubOp s;
    {
      std::unique_lock<std::mutex> lk(w->mu);
      w->cv.wait(lk, [&] { return w->stop || !w->q.empty(); });
      if (w->q.empty()) return;
      s = w->q.front();
      w->q.pop_front();
    }
    int err;
    if (s.nbytes == 0) err = 0;
    else if (e->kind == kUring && w->ring_ok) err = run_uring(e, w, s);
    else if (e->kind == kAio && w->aio_ok) err = run_aio(e, w, s);
    else err = run_psync(e, s);
    if (!err) (s.write ? e->bytes_written : e->bytes_read).fetch_add(s.nbytes);
    finish_subop(e, s, err);
  }
}

int open_cached(Engine* e, const char* path, bool write, bool* direct_out) {
  std::string key = std::string(path) + (write ? "|w" : "|r");
  std::lock_guard<std::mutex> lk(e->fd_mu);
  auto it = e->fds.find(key);
  if (it != e->fds.end()) { *direct_out = e->fd_is_direct[key]; return it->second; }
  int flags = write ? (O_WRONLY | O_CREAT) : O_RDONLY;
  int fd = -1;
  bool direct = false;
  if (e->want_direct) {
    fd = open(path, flags | O_DIRECT, 0644);
    direct = fd >= 0;
  }
  if (fd < 0) fd = open(path, flags, 0644);   // e.g. tmpfs rejects O_DIRECT with EINVAL
  if (fd < 0) return -errno;
  e->fds[key] = fd;
  e->fd_is_direct[key] = direct;
  *direct_out = direct;
  return fd;
}

}  // namespace

extern "C" {

// engine_kind: 0 auto, 1 io_uring, 2 linux aio, 3 pread/pwrite.
void* ft_nvme_create(int64_t block_size, int queue_depth, int threads, int engine_kind,
                     int use_odirect) {
  if (block_size <= 0 || queue_depth <= 0 || threads <= 0) return nullptr;
  auto* e = new Engine();
  e->block_size = block_size;
  e->queue_depth = queue_depth;
  e->n_threads = threads;
  e->want_direct = use_odirect != 0;
  e->kind = engine_kind;
  for (int i = 0; i < threads; ++i) {
    auto w = std::make_unique<Worker>();
    w->eng = e;
    e->workers.push_back(std::move(w));
  }
  if (e->kind == kAuto || e->kind == kUring) {
    bool all = true;
    for (auto& w : e->workers) { w->ring_ok = w->ring.init((unsigned)queue_depth); all &= w->ring_ok; }
    if (all) e->kind = kUring;
    else {
      for (auto& w : e->workers) if (w->ring_ok) { w->ring.destroy(); w->ring_ok = false; }
      e->kind = kAio;   // io_uring is unavailable (old kernel or a seccomp filter): next engine
    }
  }
  if (e->kind == kAio) {
    bool all = true;
    for (auto& w : e->workers) {
      w->aio_ctx = 0;
      w->aio_ok = syscall(__NR_io_setup, queue_depth, &w->aio_ctx) == 0;
      all &= w->aio_ok;
    }
    if (!all) {
      for (auto& w : e->workers) if (w->aio_ok) { syscall(__NR_io_destroy, w->aio_ctx); w->aio_ok = false; }
      e->kind = kPsync;
    }
  }
  for (auto& w : e->workers) w->th = std::thread(worker_loop, w.get());
  return e;
}

int ft_nvme_engine_kind(void* h) { return h ? ((Engine*)h)->kind : -1; }

void ft_nvme_destroy(void* h) {
  if (!h) return;
  auto* e = (Engine*)h;
  for (auto& w : e->workers) {
    { std::lock_guard<std::mutex> lk(w->mu); w->stop = true; }
    w->cv.notify_all();
  }
  for (auto& w : e->workers) {
    if (w->th.joinable()) w->th.join();
    if (w->ring_ok) w->ring.destroy();
    if (w->aio_ok) syscall(__NR_io_destroy, w->aio_ctx);
  }
  for (auto& kv : e->fds) close(kv.second);
  delete e;
}

// Queue a transfer.  Returns a positive op id or a negative errno.
int64_t ft_nvme_submit(void* h, const char* path, void* buffer, int64_t nbytes, int64_t file_offset,
                       int is_write) {
  if (!h || !path || (!buffer && nbytes) || nbytes < 0 || file_offset < 0) return -EINVAL;
  auto* e = (Engine*)h;
  bool direct = false;
  int fd = open_cached(e, path, is_write != 0, &direct);
  if (fd < 0) return fd;
  if (direct && (((uintptr_t)buffer | (uint64_t)nbytes | (uint64_t)file_offset) & 511)) {
    // misaligned request on an O_DIRECT descriptor: use a buffered descriptor instead
    std::string key = std::string(path) + (is_write ? "|wb" : "|rb");
    std::lock_guard<std::mutex> lk(e->fd_mu);
    auto it = e->fds.find(key);
    if (it == e->fds.end()) {
      int f2 = open(path, is_write ? (O_WRONLY | O_CREAT) : O_RDONLY, 0644);
      if (f2 < 0) return -errno;
      e->fds[key] = f2; e->fd_is_direct[key] = false; fd = f2;
    } else fd = it->second;
  }
  int parts = e->n_threads;
  auto st = std::make_shared<OpState>();
  int64_t id;
  // split on block boundaries
  int64_t blocks = (nbytes + e->block_size - 1) / e->block_size;
  if (blocks < parts) parts = blocks > 0 ? (int)blocks : 1;
  st->remaining.store(parts);
  {
    std::lock_guard<std::mutex> lk(e->op_mu);
    id = e->next_op++;
    e->ops[id] = st;
  }
  int64_t cursor = 0;
  for (int t = 0; t < parts; ++t) {
    int64_t share = (blocks * (t + 1) / parts - blocks * t / parts) * e->block_size;
    if (cursor + share > nbytes || t == parts - 1) share = nbytes - cursor;
    SubOp s{id, is_write != 0, fd, (char*)buffer + cursor, share, file_offset + cursor};
    cursor += share;
    Worker* w = e->workers[t].get();
    { std::lock_guard<std::mutex> lk(w->mu); w->q.push_back(s); }
    w->cv.notify_one();
  }
  return id;
}

// Block until op `id` is finished; returns 0 or its negative errno.
int ft_nvme_wait_op(void* h, int64_t id) {
  if (!h) return -EINVAL;
  auto* e = (Engine*)h;
  std::unique_lock<std::mutex> lk(e->op_mu);
  auto it = e->ops.find(id);
  if (it == e->ops.end()) return -ENOENT;
  auto st = it->second;
  e->op_cv.wait(lk, [&] { return st->remaining.load() == 0; });
  int err = st->error.load();
  e->ops.erase(id);
  return err;
}

// Block until every queued op is finished.  Returns how many ops completed
// since the previous call, or the first negative errno met.
int64_t ft_nvme_wait(void* h) {
  if (!h) return -EINVAL;
  auto* e = (Engine*)h;
  std::unique_lock<std::mutex> lk(e->op_mu);
  e->op_cv.wait(lk, [&] {
    for (auto& kv : e->ops) if (kv.second->remaining.load() != 0) return false;
    return true;
  });
  int64_t n = e->completed_since_wait;
  int err = e->first_error;
  e->completed_since_wait = 0;
  e->first_error = 0;
  e->ops.clear();
  return err ? (int64_t)err : n;
}

int ft_nvme_pending(void* h) {
  if (!h) return -EINVAL;
  auto* e = (Engine*)h;
  std::lock_guard<std::mutex> lk(e->op_mu);
  int n = 0;
  for (auto& kv : e->ops) n += kv.second->remaining.load() != 0;
  return n;
}

// One-shot blocking transfer (capability parity: aio_read / aio_write).
int ft_nvme_sync_rw(void* h, const char* path, void* buffer, int64_t nbytes, int64_t file_offset,
                    int is_write) {
  int64_t id = ft_nvme_submit(h, path, buffer, nbytes, file_offset, is_write);
  if (id < 0) return (int)id;
  return ft_nvme_wait_op(h, id);
}

// Close cached descriptors of `path` (both modes) e.g. before deleting the file.
int ft_nvme_forget(void* h, const char* path) {
  if (!h || !path) return -EINVAL;
  auto* e = (Engine*)h;
  std::lock_guard<std::mutex> lk(e->fd_mu);
  int n = 0;
  for (const char* suffix : {"|w", "|r", "|wb", "|rb"}) {
    auto it = e->fds.find(std::string(path) + suffix);
    if (it != e->fds.end()) { close(it->second); e->fd_is_direct.erase(it->first); e->fds.erase(it); ++n; }
  }
  return n;
}

int ft_nvme_open_fds(void* h) {
  if (!h) return -EINVAL;
  auto* e = (Engine*)h;
  std::lock_guard<std::mutex> lk(e->fd_mu);
  return (int)e->fds.size();
}

// kind 1: fail with EIO, kind 2: short transfer; applies to the next `count` blocks.
void ft_nvme_inject_fault(void* h, int kind, int count) {
  if (!h) return;
  auto* e = (Engine*)h;
  e->fault_countdown.store(count);
  e->fault_kind.store(kind);
}

// Registers page-locked buffers with every io_uring worker: block transfers that lie
// inside one of them are issued as fixed-buffer requests (no per-request page pinning).
// Replaces any earlier set; n = 0 drops it.  Must be called while no operation is
// pending (-EBUSY otherwise).  Returns the number of workers that hold the
// registration - 0 when the engine does not run on io_uring or the kernel refused
// (memlock limit): transfers then simply stay ordinary requests - or a negative errno.
// The reference's engine has no counterpart (libaio has no registered buffers).
int ft_nvme_register_buffers(void* h, void* const* ptrs, const int64_t* lens, int n) {
  if (!h || n < 0 || (n > 0 && (!ptrs || !lens))) return -EINVAL;
  auto* e = (Engine*)h;
  {
    std::lock_guard<std::mutex> lk(e->op_mu);
    for (auto& kv : e->ops)
      if (kv.second->remaining.load() != 0) return -EBUSY;   // a ring is in use
  }
  constexpr int64_t kPiece = 1ll << 30;          // the kernel takes at most 1 GiB per entry
  std::vector<iovec> pieces;
  for (int i = 0; i < n; ++i) {
    if (!ptrs[i] || lens[i] <= 0) return -EINVAL;
    for (int64_t off = 0; off < lens[i]; off += kPiece) {
      iovec v;
      v.iov_base = (char*)ptrs[i] + off;
      v.iov_len = (size_t)(lens[i] - off < kPiece ? lens[i] - off : kPiece);
      pieces.push_back(v);
    }
  }
  if (pieces.size() > 1024) return -E2BIG;
  for (auto& w : e->workers) w->ring_registered.store(false);
  {
    std::lock_guard<std::mutex> lk(e->reg_mu);
    e->reg = pieces;
  }
  int holders = 0;
  if (e->kind == kUring) {
    for (auto& w : e->workers) {
      if (!w->ring_ok) continue;
      if (w->ring.register_buffers(pieces.data(), (unsigned)pieces.size()) == 0 && !pieces.empty()) {
        w->ring_registered.store(true);
        ++holders;
      }
    }
  }
  return holders;
}

// Block requests issued as fixed-buffer requests so far.
int64_t ft_nvme_fixed_ops(void* h) { return h ? ((Engine*)h)->fixed_ops.load() : 0; }

void ft_nvme_stats(void* h, int64_t* bytes_read, int64_t* bytes_written) {
  if (!h) return;
  auto* e = (Engine*)h;
  if (bytes_read) *bytes_read = e->bytes_read.load();
  if (bytes_written) *bytes_written = e->bytes_written.load();
}

}  // extern "C"
