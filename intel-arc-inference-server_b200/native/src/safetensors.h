// Read-only safetensors shard: mmap, header parse, bounds checks.
//
// As the reference's reader (src/loader/safetensors.h:25-59, docs/13-loader.md:81-93): the file
// is mapped, never copied; the 8-byte header length is checked against the file size before it is
// trusted; every tensor's byte range is checked against the data section; the pages are dropped
// from the page cache on close so a 20 GB checkpoint does not stay resident twice.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.h"

namespace b2host {

struct TensorInfo {
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range inside the data section
};

class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0) fail("fstat failed");
    size_ = (uint64_t)st.st_size;
    if (size_ < 8) fail("file is shorter than its header length field");
    base_ = (const uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (base_ == MAP_FAILED) {
      base_ = nullptr;
      fail("mmap failed");
    }
    uint64_t hlen = 0;
    memcpy(&hlen, base_, 8);
    if (hlen > size_ - 8 || hlen > (1ull << 30)) fail("header length exceeds the file");  // overflow-safe
    data_off_ = 8 + hlen;
    Json h;
    if (!Json::try_parse(std::string((const char*)base_ + 8, hlen), h) || !h.is_object()) fail("header is not JSON");
    const uint64_t data_size = size_ - data_off_;
    for (const auto& m : h.members()) {
      if (m.first == "__metadata__") {
        if (m.second.is_object())
          for (const auto& kv : m.second.members())
            if (kv.second.is_string()) metadata_[kv.first] = kv.second.as_string();
        continue;
      }
      TensorInfo t;
      t.dtype = m.second.at("dtype").as_string();
      for (const Json& d : m.second.at("shape").items()) t.shape.push_back(d.as_int());
      const Json& off = m.second.at("data_offsets");
      t.begin = (uint64_t)off[0].as_int();
      t.end = (uint64_t)off[1].as_int();
      if (t.begin > t.end || t.end > data_size) fail("tensor " + m.first + " lies outside the data section");
      uint64_t n = dtype_size(t.dtype);
      for (int64_t d : t.shape) {
        if (d < 0) fail("negative dimension in " + m.first);
        n *= (uint64_t)d;
      }
      if (n != t.end - t.begin) fail("tensor " + m.first + ": shape and byte range disagree");
      names_.push_back(m.first);
      tensors_[m.first] = t;
    }
  }
  ~SafetensorsFile() {
    if (base_) {
      munmap((void*)base_, size_);
#ifdef POSIX_FADV_DONTNEED
      posix_fadvise(fd_, 0, 0, POSIX_FADV_DONTNEED);
#endif
    }
    if (fd_ >= 0) ::close(fd_);
  }
  SafetensorsFile(const SafetensorsFile&) = delete;
  SafetensorsFile& operator=(const SafetensorsFile&) = delete;

  static uint64_t dtype_size(const std::string& d) {
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    throw std::runtime_error("unknown safetensors dtype " + d);
  }
  const std::vector<std::string>& names() const { return names_; }
  bool has(const std::string& n) const { return tensors_.count(n) != 0; }
  const TensorInfo& info(const std::string& n) const {
    auto it = tensors_.find(n);
    if (it == tensors_.end()) throw std::out_of_range("no tensor " + n + " in " + path_);
    return it->second;
  }
  const uint8_t* data(const std::string& n) const { return base_ + data_off_ + info(n).begin; }
  uint64_t nbytes(const std::string& n) const { return info(n).end - info(n).begin; }
  const std::map<std::string, std::string>& metadata() const { return metadata_; }
  const std::string& path() const { return path_; }

 private:
  [[noreturn]] void fail(const std::string& why) {
    if (base_) munmap((void*)base_, size_);
    base_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
    throw std::runtime_error("safetensors " + path_ + ": " + why);
  }
  std::string path_;
  int fd_ = -1;
  uint64_t size_ = 0, data_off_ = 0;
  const uint8_t* base_ = nullptr;
  std::vector<std::string> names_;
  std::map<std::string, TensorInfo> tensors_;
  std::map<std::string, std::string> metadata_;
};

}  // namespace b2host
