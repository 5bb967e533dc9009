// GGUF version 3 reader (see gguf_file.h). The format: magic "GGUF", version, tensor count, metadata count; the
// metadata pairs (a string key, a type, a value); the tensor table (name, dimensions, ggml type, offset into the data);
// padding to general.alignment (32 unless the file says otherwise); the data.
#include "gguf_file.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "formats.h"

namespace moe {

namespace {

enum : uint32_t { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

// A cursor over the mapped header; every read checks the file's end.
struct Cursor {
  const uint8_t *p, *end;
  template <class T>
  T take() {
    if ((size_t)(end - p) < sizeof(T)) throw std::runtime_error("the file ends inside its header");
    T v;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string take_string() {
    const uint64_t n = take<uint64_t>();
    if ((uint64_t)(end - p) < n) throw std::runtime_error("the file ends inside a string");
    std::string s((const char *)p, (size_t)n);
    p += n;
    return s;
  }
  void skip(uint64_t n) {
    if ((uint64_t)(end - p) < n) throw std::runtime_error("the file ends inside a value");
    p += n;
  }
};

uint32_t scalar_size(uint32_t type) {
  switch (type) {
    case T_U8: case T_I8: case T_BOOL: return 1;
    case T_U16: case T_I16: return 2;
    case T_U32: case T_I32: case T_F32: return 4;
    case T_U64: case T_I64: case T_F64: return 8;
    default: return 0;
  }
}

}  // namespace

uint64_t gguf_type_bytes(uint32_t type, uint64_t elements) {
  if (type == GGML_F32) return elements * 4;
  if (type == GGML_F16 || type == GGML_BF16) return elements * 2;
  if (!type_known(type) || elements % block_values(type)) return 0;
  return elements / block_values(type) * block_bytes(type);
}

GgufFile::GgufFile(const std::string &path) : path_(path) {
  fd_ = ::open(path.c_str(), O_RDONLY);
  if (fd_ < 0) throw std::runtime_error("cannot open " + path + ": " + std::strerror(errno));
  struct stat st {};
  if (::fstat(fd_, &st) != 0 || st.st_size < 24) {
    ::close(fd_);
    throw std::runtime_error(path + " is too short to be a GGUF file");
  }
  size_ = (uint64_t)st.st_size;
  void *m = ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
  if (m == MAP_FAILED) {
    ::close(fd_);
    throw std::runtime_error("cannot map " + path + ": " + std::strerror(errno));
  }
  base_ = (const uint8_t *)m;
  try {
    Cursor c{base_, base_ + size_};
    if (c.take<uint32_t>() != 0x46554747u) throw std::runtime_error("not a GGUF file (magic)");
    const uint32_t version = c.take<uint32_t>();
    if (version != 3) throw std::runtime_error("GGUF version " + std::to_string(version) + ": only version 3 is read");
    const uint64_t ntensors = c.take<uint64_t>(), nmeta = c.take<uint64_t>();
    for (uint64_t i = 0; i < nmeta; i++) {
      const std::string key = c.take_string();
      const uint32_t type = c.take<uint32_t>();
      switch (type) {
        case T_U8: ints_[key] = c.take<uint8_t>(); break;
        case T_I8: ints_[key] = c.take<int8_t>(); break;
        case T_U16: ints_[key] = c.take<uint16_t>(); break;
        case T_I16: ints_[key] = c.take<int16_t>(); break;
        case T_U32: ints_[key] = c.take<uint32_t>(); break;
        case T_I32: ints_[key] = c.take<int32_t>(); break;
        case T_U64: ints_[key] = (int64_t)c.take<uint64_t>(); break;
        case T_I64: ints_[key] = c.take<int64_t>(); break;
        case T_BOOL: ints_[key] = c.take<uint8_t>() != 0; break;
        case T_F32: floats_[key] = c.take<float>(); break;
        case T_F64: floats_[key] = c.take<double>(); break;
        case T_STRING: strings_[key] = c.take_string(); break;
        case T_ARRAY: {
          const uint32_t et = c.take<uint32_t>();
          const uint64_t n = c.take<uint64_t>();
          if (et == T_STRING) {
            for (uint64_t j = 0; j < n; j++) c.take_string();
          } else if (scalar_size(et)) {
            c.skip(n * scalar_size(et));
          } else {
            throw std::runtime_error("metadata array of an unknown element type at " + key);
          }
          break;
        }
        default: throw std::runtime_error("metadata value of an unknown type at " + key);
      }
    }
    tensors_.reserve((size_t)ntensors);
    for (uint64_t i = 0; i < ntensors; i++) {
      GgufTensorInfo t;
      t.name = c.take_string();
      const uint32_t nd = c.take<uint32_t>();
      if (nd == 0 || nd > 8) throw std::runtime_error("tensor " + t.name + " has " + std::to_string(nd) + " dimensions");
      for (uint32_t d = 0; d < nd; d++) t.shape.push_back(c.take<uint64_t>());
      t.type = c.take<uint32_t>();
      t.offset = c.take<uint64_t>();  // from the data's start, fixed up below
      t.bytes = gguf_type_bytes(t.type, t.elements());
      index_[t.name] = tensors_.size();
      tensors_.push_back(std::move(t));
    }
    const uint64_t align = (uint64_t)get_int("general.alignment", 32);
    if (align == 0 || (align & (align - 1))) throw std::runtime_error("general.alignment is not a power of two");
    const uint64_t data0 = ((uint64_t)(c.p - base_) + align - 1) / align * align;
    for (GgufTensorInfo &t : tensors_) {
      t.offset += data0;
      // A tensor of a type this library does not read keeps bytes 0 and no data: it is listed, not usable.
      if (t.bytes) {
        if (t.offset + t.bytes > size_) throw std::runtime_error("tensor " + t.name + " runs past the file's end");
        t.data = base_ + t.offset;
      }
    }
  } catch (...) {
    ::munmap((void *)base_, size_);
    ::close(fd_);
    throw;
  }
}

GgufFile::~GgufFile() {
  if (base_) ::munmap((void *)base_, size_);
  if (fd_ >= 0) ::close(fd_);
}

const GgufTensorInfo *GgufFile::find(const std::string &name) const {
  auto it = index_.find(name);
  return it == index_.end() ? nullptr : &tensors_[it->second];
}

const GgufTensorInfo &GgufFile::tensor(const std::string &name) const {
  const GgufTensorInfo *t = find(name);
  if (!t) throw std::runtime_error("the file has no tensor " + name);
  if (!t->data) throw std::runtime_error("tensor " + name + " is of ggml type " + std::to_string(t->type) + ", which this library does not read");
  return *t;
}

int64_t GgufFile::get_int(const std::string &key, int64_t otherwise) const {
  auto it = ints_.find(key);
  return it == ints_.end() ? otherwise : it->second;
}

double GgufFile::get_float(const std::string &key, double otherwise) const {
  auto it = floats_.find(key);
  return it == floats_.end() ? otherwise : it->second;
}

std::string GgufFile::get_string(const std::string &key, const std::string &otherwise) const {
  auto it = strings_.find(key);
  return it == strings_.end() ? otherwise : it->second;
}

int64_t GgufFile::arch_int(const std::string &suffix, int64_t otherwise) const {
  const std::string arch = get_string("general.architecture");
  return arch.empty() ? otherwise : get_int(arch + "." + suffix, otherwise);
}

std::vector<float> gguf_to_f32(const GgufTensorInfo &t) {
  const uint64_t n = t.elements();
  std::vector<float> out((size_t)n);
  if (t.type == GGML_F32) {
    std::memcpy(out.data(), t.data, n * 4);
  } else if (t.type == GGML_BF16) {
    for (uint64_t i = 0; i < n; i++) {
      uint16_t h;
      std::memcpy(&h, t.data + 2 * i, 2);
      const uint32_t u = (uint32_t)h << 16;
      std::memcpy(&out[i], &u, 4);
    }
  } else if (t.type == GGML_F16) {
    for (uint64_t i = 0; i < n; i++) {
      uint16_t h;
      std::memcpy(&h, t.data + 2 * i, 2);
      const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, ex = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
      uint32_t u;
      if (ex == 0) {
        if (man == 0) {
          u = sign;
        } else {  // subnormal: renormalise
          int e = -1;
          uint32_t m = man;
          do {
            m <<= 1, e++;
          } while (!(m & 0x400u));
          u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
      } else if (ex == 31) {
        u = sign | 0x7F800000u | (man << 13);
      } else {
        u = sign | ((ex + 127 - 15) << 23) | (man << 13);
      }
      std::memcpy(&out[i], &u, 4);
    }
  } else {
    throw std::runtime_error("tensor " + t.name + " is not F32, F16 or BF16");
  }
  return out;
}

}  // namespace moe
