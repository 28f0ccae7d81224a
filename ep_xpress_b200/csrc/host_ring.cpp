// Bounded single-producer / multi-reader ring in POSIX shared memory: the wire of the
// host-staged `host_ce` transport.
//
// Same contract as the reference's file-backed ring (ep_xpress/ring.py:1-261): a fixed
// number of payload slots, each going FREE -> WRITING -> READY -> FREE; a READY slot carries
// a generation id and the bitmask of ranks that must read it; readers acknowledge with
// their bit and only the LAST expected reader frees the slot, so a slow reader blocks its
// own slot and nothing else; a stale generation never satisfies a wait; a sticky abort
// word ends every wait. The reference serialises its control words with fcntl locks from
// Python; here they are lock-free std::atomic words with acquire/release ordering, one
// writer per word except the acknowledgement mask, which is a fetch_or.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <torch/extension.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <stdexcept>
#include <string>

namespace py = pybind11;

namespace epx {
namespace {

constexpr uint64_t kMagic = 0x4550584252494e47ull;   // "EPXBRING"
constexpr uint64_t kFree = 0, kWriting = 1, kReady = 2;
constexpr size_t kHeaderBytes = 4096;
constexpr size_t kSlotControlBytes = 64;

struct RingHeader {
  uint64_t magic;
  uint64_t slots;
  uint64_t slot_bytes;
  std::atomic<uint64_t> aborted;
};

struct SlotControl {
  std::atomic<uint64_t> state;
  std::atomic<int64_t> generation;
  std::atomic<uint64_t> expected;
  std::atomic<uint64_t> acked;
  std::atomic<uint64_t> rows;
  uint64_t pad[3];
};
static_assert(sizeof(SlotControl) == kSlotControlBytes, "one cache line per slot control block");

class HostRing {
 public:
  HostRing(const std::string& path, int64_t slots, int64_t slot_bytes, bool create) : path_(path) {
    if (create && (slots <= 0 || slot_bytes <= 0)) throw std::invalid_argument("slots and slot_bytes must be positive");
    const int flags = create ? (O_RDWR | O_CREAT | O_EXCL) : O_RDWR;
    fd_ = ::open(path.c_str(), flags, 0600);
    if (fd_ < 0) throw std::runtime_error("cannot open ring file " + path + ": " + std::strerror(errno));
    if (create) {
      slot_stride_ = (static_cast<size_t>(slot_bytes) + 4095) / 4096 * 4096;
      bytes_ = kHeaderBytes + static_cast<size_t>(slots) * kSlotControlBytes;
      bytes_ = (bytes_ + 4095) / 4096 * 4096;
      payload_offset_ = bytes_;
      bytes_ += static_cast<size_t>(slots) * slot_stride_;
      if (::ftruncate(fd_, static_cast<off_t>(bytes_)) != 0) {
        ::close(fd_);
        ::unlink(path.c_str());
        throw std::runtime_error("cannot size ring file");
      }
    } else {
      struct stat st;
      if (::fstat(fd_, &st) != 0 || st.st_size < static_cast<off_t>(kHeaderBytes)) {
        ::close(fd_);
        throw std::runtime_error("ring file is too small");
      }
      bytes_ = static_cast<size_t>(st.st_size);
    }
    base_ = static_cast<unsigned char*>(::mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0));
    if (base_ == MAP_FAILED) {
      ::close(fd_);
      throw std::runtime_error("cannot map ring file");
    }
    header_ = reinterpret_cast<RingHeader*>(base_);
    if (create) {
      std::memset(base_, 0, payload_offset_);
      header_->slots = static_cast<uint64_t>(slots);
      header_->slot_bytes = static_cast<uint64_t>(slot_bytes);
      std::atomic_thread_fence(std::memory_order_release);
      header_->magic = kMagic;
    } else {
      if (header_->magic != kMagic) {
        close();
        throw std::runtime_error("not a ring file (bad magic)");
      }
      slot_stride_ = (static_cast<size_t>(header_->slot_bytes) + 4095) / 4096 * 4096;
      payload_offset_ = (kHeaderBytes + header_->slots * kSlotControlBytes + 4095) / 4096 * 4096;
      if (payload_offset_ + header_->slots * slot_stride_ > bytes_) {
        close();
        throw std::runtime_error("ring file is truncated");
      }
    }
    owner_ = create;
  }

  ~HostRing() { close(); }

  void close() {
    if (base_ != nullptr && base_ != MAP_FAILED) ::munmap(base_, bytes_);
    base_ = nullptr;
    header_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }
  void unlink() { ::unlink(path_.c_str()); }

  int64_t slots() const { return static_cast<int64_t>(live()->slots); }
  int64_t slot_bytes() const { return static_cast<int64_t>(live()->slot_bytes); }

  // Producer: claim a FREE slot for `generation`, to be read by the ranks in `expected_mask`.
  // Returns the slot index or -1 when every slot is still in use.
  int64_t try_claim(int64_t generation, uint64_t expected_mask) {
    check_abort();
    if (expected_mask == 0) throw std::invalid_argument("a chunk needs at least one reader");
    const uint64_t n = live()->slots;
    for (uint64_t i = 0; i < n; ++i) {
      const uint64_t slot = (cursor_ + i) % n;
      SlotControl* c = control(slot);
      uint64_t expect = kFree;
      if (c->state.compare_exchange_strong(expect, kWriting, std::memory_order_acquire)) {
        c->generation.store(generation, std::memory_order_relaxed);
        c->expected.store(expected_mask, std::memory_order_relaxed);
        c->acked.store(0, std::memory_order_relaxed);
        c->rows.store(0, std::memory_order_relaxed);
        cursor_ = slot + 1;
        return static_cast<int64_t>(slot);
      }
    }
    return -1;
  }

  void publish(int64_t slot, int64_t rows) {
    SlotControl* c = control(slot);
    if (c->state.load(std::memory_order_relaxed) != kWriting) throw std::runtime_error("slot is not being written");
    c->rows.store(static_cast<uint64_t>(rows), std::memory_order_relaxed);
    c->state.store(kReady, std::memory_order_release);
  }

  // Reader: rows of the slot if it is READY with exactly this generation, else -1.
  int64_t ready(int64_t slot, int64_t generation) {
    check_abort();
    SlotControl* c = control(slot);
    if (c->state.load(std::memory_order_acquire) != kReady) return -1;
    if (c->generation.load(std::memory_order_relaxed) != generation) return -1;
    return static_cast<int64_t>(c->rows.load(std::memory_order_relaxed));
  }

  // Reader `rank` is done with (slot, generation). Returns true when this freed the slot.
  bool ack(int64_t slot, int64_t generation, int rank) {
    SlotControl* c = control(slot);
    if (rank < 0 || rank >= 64) throw std::invalid_argument("reader rank out of range");
    const uint64_t bit = 1ull << rank;
    if (c->state.load(std::memory_order_acquire) != kReady ||
        c->generation.load(std::memory_order_relaxed) != generation)
      throw std::runtime_error("stale acknowledgement: the slot holds another generation");
    const uint64_t expected = c->expected.load(std::memory_order_relaxed);
    if (!(expected & bit)) throw std::runtime_error("this rank is not an expected reader of the slot");
    const uint64_t before = c->acked.fetch_or(bit, std::memory_order_acq_rel);
    if (before & bit) throw std::runtime_error("duplicate acknowledgement");
    if ((before | bit) == expected) {
      c->state.store(kFree, std::memory_order_release);
      return true;
    }
    return false;
  }

  py::tuple snapshot(int64_t slot) {
    SlotControl* c = control(slot);
    return py::make_tuple(c->state.load(), c->generation.load(), c->expected.load(), c->acked.load(), c->rows.load());
  }

  void abort() { live()->aborted.store(1, std::memory_order_release); }
  bool aborted() const { return live()->aborted.load(std::memory_order_acquire) != 0; }

  // uint8 CPU tensor over the slot's payload; valid while this object is open.
  at::Tensor payload(int64_t slot) {
    control(slot);
    return at::from_blob(base_ + payload_offset_ + static_cast<size_t>(slot) * slot_stride_,
                         {static_cast<int64_t>(live()->slot_bytes)}, at::TensorOptions().dtype(at::kByte));
  }

 private:
  RingHeader* live() const {
    if (header_ == nullptr) throw std::runtime_error("the ring is closed");
    return header_;
  }
  SlotControl* control(int64_t slot) const {
    if (slot < 0 || static_cast<uint64_t>(slot) >= live()->slots) throw std::out_of_range("slot index out of range");
    return reinterpret_cast<SlotControl*>(base_ + kHeaderBytes) + slot;
  }
  void check_abort() const {
    if (aborted()) throw std::runtime_error("the ring was aborted by a peer");
  }

  std::string path_;
  int fd_ = -1;
  unsigned char* base_ = nullptr;
  RingHeader* header_ = nullptr;
  size_t bytes_ = 0, slot_stride_ = 0, payload_offset_ = 0;
  uint64_t cursor_ = 0;
  bool owner_ = false;
};

}  // namespace

void bind_host_ring(py::module_& m) {
  py::class_<HostRing>(m, "HostRing")
      .def(py::init<const std::string&, int64_t, int64_t, bool>(), py::arg("path"), py::arg("slots") = 0,
           py::arg("slot_bytes") = 0, py::arg("create") = false)
      .def("slots", &HostRing::slots)
      .def("slot_bytes", &HostRing::slot_bytes)
      .def("try_claim", &HostRing::try_claim)
      .def("publish", &HostRing::publish)
      .def("ready", &HostRing::ready)
      .def("ack", &HostRing::ack)
      .def("snapshot", &HostRing::snapshot)
      .def("abort", &HostRing::abort)
      .def("aborted", &HostRing::aborted)
      .def("payload", &HostRing::payload)
      .def("unlink", &HostRing::unlink)
      .def("close", &HostRing::close);
}

}  // namespace epx
