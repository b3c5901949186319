// safetensors.cu — checkpoint blocks straight into device weight storage.
//
// Replaces the weight part of SafeTensorsReader::load (Serialization/SafeTensorsReader.cpp:276-325): for
// every layer that owns parameters the tensor "<layer name>/weights" (dtype F32, any shape whose element
// count equals the layer's params_count) is the layer's flat weight block.  The reference reads it into the
// host weight block; here the file is streamed through two pinned staging buffers into the layer's device
// block, so no host copy of the model is ever held.  File layout (the safetensors container the reference's
// writer produces, SafeTensorsWriter.cpp:244-300): 8-byte little-endian header length, a JSON header mapping
// tensor name -> {dtype, shape, data_offsets [begin, end)} relative to the end of the header, then the data.
// Other tensors (tokenizer/json, encoder blobs, optimizer state) are skipped.  BF16 tensors are accepted and
// widened to fp32 on the device.
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace mb {
namespace {

struct StTensor {
  std::string dtype;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;
  uint64_t elements() const {
    uint64_t n = 1;
    for (uint64_t d : shape) n *= d;
    return n;
  }
};

// Minimal JSON reader for the header: objects, arrays, strings (with escapes), numbers, literals.
struct Json {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() {
    while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < e && *p == c) { ++p; return true; }
    return false;
  }
  bool string(std::string* out) {
    ws();
    if (p >= e || *p != '"') return ok = false;
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        char c = *p;
        if (c == 'u') {  // \uXXXX: keep names ASCII-comparable, anything else becomes '?'
          unsigned v = 0;
          for (int i = 1; i <= 4 && p + i < e; ++i) {
            const char h = p[i];
            v = v * 16 + (h >= '0' && h <= '9' ? h - '0' : (h | 32) >= 'a' && (h | 32) <= 'f' ? (h | 32) - 'a' + 10 : 0);
          }
          p += 4;
          c = v < 128 ? static_cast<char>(v) : '?';
        } else if (c == 'n') c = '\n';
        else if (c == 't') c = '\t';
        else if (c == 'r') c = '\r';
        else if (c == 'b') c = '\b';
        else if (c == 'f') c = '\f';
        if (out) out->push_back(c);
        ++p;
      } else {
        if (out) out->push_back(*p);
        ++p;
      }
    }
    if (p >= e) return ok = false;
    ++p;
    return true;
  }
  bool number(uint64_t* out) {
    ws();
    const char* s = p;
    uint64_t v = 0;
    while (p < e && *p >= '0' && *p <= '9') v = v * 10 + static_cast<uint64_t>(*p++ - '0');
    if (p == s) return ok = false;
    if (out) *out = v;
    return true;
  }
  bool skip() {  // any value
    ws();
    if (p >= e) return ok = false;
    if (*p == '"') return string(nullptr);
    if (*p == '{' || *p == '[') {
      const char close = *p == '{' ? '}' : ']';
      const bool obj = *p == '{';
      ++p;
      if (eat(close)) return true;
      do {
        if (obj) {
          if (!string(nullptr) || !eat(':')) return ok = false;
        }
        if (!skip()) return false;
      } while (eat(','));
      return eat(close) ? true : (ok = false);
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n') ++p;  // number / true / false / null
    return true;
  }
};

bool parse_header(const std::string& text, std::map<std::string, StTensor>* out) {
  Json j{text.data(), text.data() + text.size()};
  if (!j.eat('{')) return false;
  if (j.eat('}')) return true;
  do {
    std::string name;
    if (!j.string(&name) || !j.eat(':')) return false;
    j.ws();
    if (name == "__metadata__" || j.p >= j.e || *j.p != '{') {
      if (!j.skip()) return false;
      continue;
    }
    ++j.p;
    StTensor t;
    bool have_off = false;
    if (!j.eat('}')) {
      do {
        std::string key;
        if (!j.string(&key) || !j.eat(':')) return false;
        if (key == "dtype") {
          if (!j.string(&t.dtype)) return false;
        } else if (key == "shape" || key == "data_offsets") {
          std::vector<uint64_t> v;
          if (!j.eat('[')) return false;
          if (!j.eat(']')) {
            do {
              uint64_t x;
              if (!j.number(&x)) return false;
              v.push_back(x);
            } while (j.eat(','));
            if (!j.eat(']')) return false;
          }
          if (key == "shape") t.shape = v;
          else {
            if (v.size() != 2 || v[1] < v[0]) return false;
            t.begin = v[0]; t.end = v[1];
            have_off = true;
          }
        } else if (!j.skip()) {
          return false;
        }
      } while (j.eat(','));
      if (!j.eat('}')) return false;
    }
    if (have_off) (*out)[name] = t;
  } while (j.eat(','));
  return j.eat('}') && j.ok;
}

__global__ void widen_bf16_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}

struct File {
  FILE* f = nullptr;
  ~File() { if (f) fclose(f); }
};

// Two pinned staging buffers: the read of chunk i+1 from the file overlaps the H2D copy of chunk i.
struct Staging {
  static constexpr size_t BYTES = size_t(32) << 20;
  void* buf[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  cudaStream_t st = nullptr;
  int init() {
    MB_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      MB_CUDA(cudaMallocHost(&buf[i], BYTES));
      MB_CUDA(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
    }
    return MIMIR_B200_OK;
  }
  ~Staging() {
    for (int i = 0; i < 2; ++i) {
      if (done[i]) cudaEventDestroy(done[i]);
      if (buf[i]) cudaFreeHost(buf[i]);
    }
    if (st) cudaStreamDestroy(st);
  }
};

int stream_to_device(FILE* f, uint64_t file_off, uint64_t bytes, void* dev, Staging& s, const char* what) {
  if (fseeko(f, static_cast<off_t>(file_off), SEEK_SET) != 0) return fail(MIMIR_B200_E_INVALID, "safetensors: seek failed for %s", what);
  uint64_t done = 0;
  int k = 0;
  while (done < bytes) {
    const size_t n = static_cast<size_t>(std::min<uint64_t>(Staging::BYTES, bytes - done));
    MB_CUDA(cudaEventSynchronize(s.done[k]));  // the copy that last used this buffer has finished
    if (fread(s.buf[k], 1, n, f) != n) return fail(MIMIR_B200_E_INVALID, "safetensors: file truncated while reading %s", what);
    MB_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dev) + done, s.buf[k], n, cudaMemcpyHostToDevice, s.st));
    MB_CUDA(cudaEventRecord(s.done[k], s.st));
    done += n;
    k ^= 1;
  }
  return MIMIR_B200_OK;
}

}  // namespace
}  // namespace mb

extern "C" {

using namespace mb;

int mimir_b200_model_load_safetensors(MimirB200ModelHandle m, const char* path, int strict, int* layers_loaded,
                                      unsigned long long* bytes_loaded) {
  DeviceScope dev_scope(model_device(m));
  if (!ctx().initialised) return fail(MIMIR_B200_E_NOT_INIT, "mimir_b200_init has not been called");
  if (!m || !path) return fail(MIMIR_B200_E_INVALID, "load_safetensors: null argument");
  if (layers_loaded) *layers_loaded = 0;
  if (bytes_loaded) *bytes_loaded = 0;
  File file;
  file.f = fopen(path, "rb");
  if (!file.f) return fail(MIMIR_B200_E_INVALID, "load_safetensors: cannot open %s", path);
  unsigned char lenb[8];
  if (fread(lenb, 1, 8, file.f) != 8) return fail(MIMIR_B200_E_INVALID, "load_safetensors: %s is shorter than a header", path);
  uint64_t hlen = 0;
  for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | lenb[i];
  if (fseeko(file.f, 0, SEEK_END) != 0) return fail(MIMIR_B200_E_INVALID, "load_safetensors: seek failed");
  const uint64_t fsize = static_cast<uint64_t>(ftello(file.f));
  if (hlen == 0 || hlen > (uint64_t(1) << 30) || 8 + hlen > fsize) return fail(MIMIR_B200_E_INVALID, "load_safetensors: bad header length in %s", path);
  std::string header(hlen, '\0');
  fseeko(file.f, 8, SEEK_SET);
  if (fread(&header[0], 1, hlen, file.f) != hlen) return fail(MIMIR_B200_E_INVALID, "load_safetensors: header truncated");
  std::map<std::string, StTensor> tensors;
  if (!parse_header(header, &tensors)) return fail(MIMIR_B200_E_INVALID, "load_safetensors: header of %s is not valid JSON", path);
  const uint64_t data0 = 8 + hlen;

  int n_layers = 0;
  MB_TRY(mimir_b200_model_num_layers(m, &n_layers));
  // Pass 1: check every tensor that will be loaded - dtype, element count without overflow, offsets against the
  // file size without wrap-around - before any layer's device weights are touched.  The header is untrusted input.
  struct Job { int layer; uint64_t begin, elems; bool f32; std::string name; };
  std::vector<Job> jobs;
  const uint64_t data_bytes = fsize - data0;
  for (int li = 0; li < n_layers; ++li) {
    const char* lname = nullptr;
    uint64_t params = 0;
    MB_TRY(mimir_b200_model_layer_info(m, li, &lname, &params));
    if (params == 0) continue;  // "Layer has no weights"
    const std::string tname = std::string(lname) + "/weights";
    auto it = tensors.find(tname);
    if (it == tensors.end()) {
      if (strict) return fail(MIMIR_B200_E_INVALID, "Missing tensor in strict mode: %s", tname.c_str());
      continue;
    }
    const StTensor& t = it->second;
    const bool f32 = t.dtype == "F32", bf16 = t.dtype == "BF16";
    if (!f32 && !bf16) return fail(MIMIR_B200_E_UNSUPPORTED, "load_safetensors: %s has dtype %s (F32 or BF16 expected)", tname.c_str(), t.dtype.c_str());
    uint64_t elems = 1;
    bool overflow = false;
    for (uint64_t d : t.shape) {
      if (d != 0 && elems > (uint64_t(1) << 62) / d) { overflow = true; break; }
      elems *= d;
    }
    const uint64_t esz = f32 ? 4 : 2;
    if (overflow || elems != params)
      return fail(MIMIR_B200_E_INVALID, "Size mismatch for %s: expected %llu got %llu", tname.c_str(), static_cast<unsigned long long>(params),
                  static_cast<unsigned long long>(overflow ? ~0ull : elems));
    if (t.end < t.begin || t.end > data_bytes || t.end - t.begin != elems * esz)
      return fail(MIMIR_B200_E_INVALID, "load_safetensors: data_offsets of %s do not match its shape or the file size", tname.c_str());
    jobs.push_back(Job{li, t.begin, elems, f32, tname});
  }
  // Pass 2: stream the checked tensors into the layers' device blocks.
  Staging stg;
  MB_TRY(stg.init());
  int loaded = 0;
  unsigned long long total = 0;
  for (const Job& jb : jobs) {
    const uint64_t elems = jb.elems, esz = jb.f32 ? 4 : 2;
    float* dev = nullptr;
    MB_TRY(mimir_b200_model_weights_device(m, jb.layer, elems, &dev));
    if (jb.f32) {
      MB_TRY(stream_to_device(file.f, data0 + jb.begin, elems * 4, dev, stg, jb.name.c_str()));
    } else {
      void* tmp = nullptr;
      MB_TRY(dev_alloc(&tmp, elems * 2, "safetensors.bf16"));
      int s = stream_to_device(file.f, data0 + jb.begin, elems * 2, tmp, stg, jb.name.c_str());
      if (s == MIMIR_B200_OK) {
        widen_bf16_kernel<<<static_cast<int>(std::min<uint64_t>((elems + 255) / 256, 148 * 16)), 256, 0, stg.st>>>(
            static_cast<const __nv_bfloat16*>(tmp), dev, static_cast<long long>(elems));
        if (cudaGetLastError() != cudaSuccess) s = fail(MIMIR_B200_E_CUDA, "safetensors: widen kernel launch failed");
        count_launch();
      }
      cudaStreamSynchronize(stg.st);
      dev_free(tmp, elems * 2);
      if (s != MIMIR_B200_OK) return s;
    }
    ++loaded;
    total += elems * esz;
  }
  MB_CUDA(cudaStreamSynchronize(stg.st));
  if (layers_loaded) *layers_loaded = loaded;
  if (bytes_loaded) *bytes_loaded = total;
  return MIMIR_B200_OK;
}

}  // extern "C"
