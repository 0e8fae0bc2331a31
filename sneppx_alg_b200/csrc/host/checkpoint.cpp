// `.sneppx` checkpoint container: writer, reader and an asynchronous double-buffered saver.
//
// Byte layout (little-endian, packed), identical to the reference's C reader/writer
// (fs/format/checkpoint_reader.h:43-67, checkpoint_reader.c:45-265) and Python twin
// (interface_bindings/checkpoint.py:10-159):
//   header  72 B : u32 magic_lo 0x41524958, u32 magic_hi 0x434B5054, u32 version 1, u32 num_tensors,
//                  u64 metadata_offset, u64 metadata_size, u64 total_size, 32 reserved bytes
//   records 152 B each : u64 shape[8], u32 ndim, u32 dtype, u64 data_offset (absolute), u64 data_size, u64 stride[8]
//   tensor data in record order, then the metadata JSON (UTF-8).
// dtype 0 is float32 (the only value the reference writes). Other element types (1 f64, 2 f16, 3 bf16, 4 i32,
// 5 i64, 6 u8, 7 fp8 e4m3) use further codes and are also named in the metadata so the reference reader, which
// only copies bytes, still opens the file.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr uint32_t kMagicLo = 0x41524958u, kMagicHi = 0x434B5054u, kVersion = 1;

#pragma pack(push, 1)
struct Header {
  uint32_t magic_lo, magic_hi, version, num_tensors;
  uint64_t metadata_offset, metadata_size, total_size;
  uint8_t reserved[32];
};
struct Record {
  uint64_t shape[8];
  uint32_t ndim, dtype;
  uint64_t data_offset, data_size;
  uint64_t stride[8];
};
#pragma pack(pop)
static_assert(sizeof(Header) == 72, "header must be 72 bytes");
static_assert(sizeof(Record) == 152, "record must be 152 bytes");

struct Reader {
  FILE* f = nullptr;
  Header h{};
  std::vector<Record> recs;
  std::string meta;
};

// strides: optional [n * 8] element strides written verbatim (the reference's Python writer stores zeros unless told
// otherwise); null -> contiguous row-major strides.
int write_file(const char* path, int n, const uint64_t* shapes, const uint32_t* ndims, const uint32_t* dtypes,
               const void* const* data, const uint64_t* nbytes, const char* meta, const uint64_t* strides = nullptr) {
  std::string tmp = std::string(path) + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return -1;
  const uint64_t meta_len = meta ? strlen(meta) : 0;
  Header h{};
  h.magic_lo = kMagicLo; h.magic_hi = kMagicHi; h.version = kVersion; h.num_tensors = (uint32_t)n;
  uint64_t off = sizeof(Header) + (uint64_t)n * sizeof(Record);
  std::vector<Record> recs((size_t)n);
  for (int i = 0; i < n; ++i) {
    Record& r = recs[i];
    memset(&r, 0, sizeof(r));
    r.ndim = ndims[i]; r.dtype = dtypes[i];
    uint64_t st = 1;
    for (int d = (int)r.ndim - 1; d >= 0; --d) {
      r.shape[d] = shapes[(size_t)i * 8 + d];
      r.stride[d] = strides ? strides[(size_t)i * 8 + d] : st;
      st *= r.shape[d];
    }
    r.data_offset = off; r.data_size = nbytes[i];
    off += nbytes[i];
  }
  h.metadata_offset = off; h.metadata_size = meta_len; h.total_size = off + meta_len;
  bool ok = fwrite(&h, sizeof(h), 1, f) == 1;
  ok = ok && (n == 0 || fwrite(recs.data(), sizeof(Record), (size_t)n, f) == (size_t)n);
  for (int i = 0; ok && i < n; ++i) ok = nbytes[i] == 0 || fwrite(data[i], 1, nbytes[i], f) == nbytes[i];
  if (ok && meta_len) ok = fwrite(meta, 1, meta_len, f) == meta_len;
  ok = (fclose(f) == 0) && ok;
  if (!ok) { remove(tmp.c_str()); return -2; }
  return rename(tmp.c_str(), path) == 0 ? 0 : -3;
}

// ---- asynchronous saver: jobs own their staging copies; one writer thread drains the queue in order
struct Job {
  std::string path, meta;
  std::vector<uint64_t> shapes, nbytes;
  std::vector<uint32_t> ndims, dtypes;
  std::vector<std::vector<uint8_t>> bufs;
};
struct Saver {
  std::thread th;
  std::mutex mu;
  std::condition_variable cv, idle;
  std::deque<Job*> q;
  bool stop = false;
  int in_flight = 0;
  std::atomic<int> errors{0};
  size_t max_pending;
  void run() {
    for (;;) {
      Job* j = nullptr;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait(lk, [&] { return stop || !q.empty(); });
        if (q.empty()) return;
        j = q.front();
        q.pop_front();
      }
      std::vector<const void*> ptrs;
      for (auto& b : j->bufs) ptrs.push_back(b.data());
      if (write_file(j->path.c_str(), (int)j->bufs.size(), j->shapes.data(), j->ndims.data(), j->dtypes.data(),
                     ptrs.data(), j->nbytes.data(), j->meta.c_str()) != 0)
        errors++;
      delete j;
      {
        std::lock_guard<std::mutex> lk(mu);
        --in_flight;
      }
      idle.notify_all();
    }
  }
};

}  // namespace

extern "C" {

int sx_ckpt_write(const char* path, int n, const uint64_t* shapes, const uint32_t* ndims, const uint32_t* dtypes,
                  const void* const* data, const uint64_t* nbytes, const char* metadata_json, const uint64_t* strides) {
  return write_file(path, n, shapes, ndims, dtypes, data, nbytes, metadata_json, strides);
}

void* sx_ckpt_open(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) return nullptr;
  Reader* r = new Reader();
  r->f = f;
  bool ok = fread(&r->h, sizeof(Header), 1, f) == 1 && r->h.magic_lo == kMagicLo && r->h.magic_hi == kMagicHi &&
            r->h.version <= kVersion && r->h.num_tensors < (1u << 24);
  // every size and offset below comes from the file: check it against the file's length before trusting it
  uint64_t file_size = 0;
  if (ok) {
    long cur = ftell(f);
    ok = cur >= 0 && fseek(f, 0, SEEK_END) == 0;
    long end = ok ? ftell(f) : -1;
    ok = ok && end >= 0 && fseek(f, cur, SEEK_SET) == 0;
    file_size = ok ? (uint64_t)end : 0;
  }
  auto in_file = [&](uint64_t off, uint64_t len) { return off <= file_size && len <= file_size - off; };
  ok = ok && in_file(sizeof(Header), (uint64_t)r->h.num_tensors * sizeof(Record));
  if (ok) {
    r->recs.resize(r->h.num_tensors);
    ok = r->h.num_tensors == 0 || fread(r->recs.data(), sizeof(Record), r->h.num_tensors, f) == r->h.num_tensors;
  }
  for (size_t i = 0; ok && i < r->recs.size(); ++i)
    ok = r->recs[i].ndim <= 8 && in_file(r->recs[i].data_offset, r->recs[i].data_size);
  ok = ok && in_file(r->h.metadata_offset, r->h.metadata_size);
  if (ok && r->h.metadata_size) {
    r->meta.resize(r->h.metadata_size);
    ok = fseek(f, (long)r->h.metadata_offset, SEEK_SET) == 0 && fread(&r->meta[0], 1, r->h.metadata_size, f) == r->h.metadata_size;
  }
  if (!ok) { fclose(f); delete r; return nullptr; }
  return r;
}
int sx_ckpt_num_tensors(void* h) { return (int)static_cast<Reader*>(h)->h.num_tensors; }
unsigned long long sx_ckpt_total_size(void* h) { return static_cast<Reader*>(h)->h.total_size; }
int sx_ckpt_tensor_info(void* h, int i, uint64_t* shape8, uint32_t* ndim, uint32_t* dtype, uint64_t* nbytes) {
  Reader* r = static_cast<Reader*>(h);
  if (i < 0 || i >= (int)r->recs.size()) return -1;
  memcpy(shape8, r->recs[i].shape, sizeof(uint64_t) * 8);
  *ndim = r->recs[i].ndim; *dtype = r->recs[i].dtype; *nbytes = r->recs[i].data_size;
  return 0;
}
int sx_ckpt_read_tensor(void* h, int i, void* dst) {
  Reader* r = static_cast<Reader*>(h);
  if (i < 0 || i >= (int)r->recs.size()) return -1;
  if (fseek(r->f, (long)r->recs[i].data_offset, SEEK_SET) != 0) return -2;
  return fread(dst, 1, r->recs[i].data_size, r->f) == r->recs[i].data_size ? 0 : -3;
}
const char* sx_ckpt_metadata(void* h) { return static_cast<Reader*>(h)->meta.c_str(); }
void sx_ckpt_close(void* h) {
  Reader* r = static_cast<Reader*>(h);
  if (r->f) fclose(r->f);
  delete r;
}

void* sx_ckpt_saver_create(int max_pending) {
  Saver* s = new Saver();
  s->max_pending = max_pending > 0 ? (size_t)max_pending : 2;  // two staging generations: save N+1 stages while N is written
  s->th = std::thread([s] { s->run(); });
  return s;
}
// Copies every tensor into the job's staging buffers (the caller may reuse its memory on return) and queues the write.
// Blocks while max_pending jobs are already waiting, which bounds host memory to max_pending checkpoints.
int sx_ckpt_saver_submit(void* hs, const char* path, int n, const uint64_t* shapes, const uint32_t* ndims,
                         const uint32_t* dtypes, const void* const* data, const uint64_t* nbytes, const char* meta) {
  Saver* s = static_cast<Saver*>(hs);
  Job* j = new Job();
  j->path = path; j->meta = meta ? meta : "";
  j->shapes.assign(shapes, shapes + (size_t)n * 8);
  j->ndims.assign(ndims, ndims + n); j->dtypes.assign(dtypes, dtypes + n); j->nbytes.assign(nbytes, nbytes + n);
  j->bufs.resize((size_t)n);
  for (int i = 0; i < n; ++i) {
    j->bufs[i].resize(nbytes[i]);
    if (nbytes[i]) memcpy(j->bufs[i].data(), data[i], nbytes[i]);
  }
  {
    std::unique_lock<std::mutex> lk(s->mu);
    s->idle.wait(lk, [&] { return (size_t)s->in_flight < s->max_pending; });
    s->q.push_back(j);
    ++s->in_flight;
  }
  s->cv.notify_one();
  return 0;
}
int sx_ckpt_saver_wait(void* hs) {
  Saver* s = static_cast<Saver*>(hs);
  std::unique_lock<std::mutex> lk(s->mu);
  s->idle.wait(lk, [&] { return s->in_flight == 0; });
  return s->errors.load();
}
void sx_ckpt_saver_destroy(void* hs) {
  Saver* s = static_cast<Saver*>(hs);
  sx_ckpt_saver_wait(hs);
  {
    std::lock_guard<std::mutex> lk(s->mu);
    s->stop = true;
  }
  s->cv.notify_all();
  s->th.join();
  delete s;
}

}  // extern "C"
