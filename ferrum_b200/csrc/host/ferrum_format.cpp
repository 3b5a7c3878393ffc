// Reader / writer of the FERRUM01 checkpoint container.
//
// Byte layout (ferrum-serialize/src/format.rs:9-48, io.rs:13-202; the header is what
// bincode 1.3 emits with its default options: little-endian, fixed-width integers,
// lengths as u64, enum variant index as u32, no padding):
//
//   "FERRUM01"                                   8 bytes
//   u64  header_len
//   header:
//     u32 version (= 1) ; u64 num_tensors ; u64 data_size ; u64 map_len
//     map_len x { u64 name_len ; name bytes ; u64 ndim ; ndim x u64 dims ;
//                 u32 dtype (0 F32,1 F64,2 F16,3 BF16,4 I32,5 I64,6 U8,7 Bool) ;
//                 u64 offset ; u64 size }
//   data section: data_size bytes, tensors back to back at their offsets.
//
// Tensors are located by offset / size, never by map order.  All eight dtypes are
// read and written (the reference materialises only F32/F64/I32/I64).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#define FB_API extern "C" __attribute__((visibility("default")))

namespace {

struct Entry {
  std::string name;
  std::vector<uint64_t> dims;
  uint32_t dtype = 0;
  uint64_t offset = 0;
  uint64_t size = 0;
};

struct Reader {
  FILE* f = nullptr;
  uint64_t data_start = 0;
  uint64_t data_size = 0;
  uint32_t version = 0;
  std::vector<Entry> entries;
};

void set_err(char* err, int errlen, const std::string& msg) {
  if (err != nullptr && errlen > 0) {
    std::snprintf(err, static_cast<size_t>(errlen), "%s", msg.c_str());
  }
}

void put_u32(std::vector<uint8_t>& b, uint32_t v) {
  for (int i = 0; i < 4; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
}
void put_u64(std::vector<uint8_t>& b, uint64_t v) {
  for (int i = 0; i < 8; ++i) b.push_back(static_cast<uint8_t>(v >> (8 * i)));
}

struct Cursor {
  const uint8_t* p;
  size_t n;
  size_t pos = 0;
  bool ok = true;
  uint32_t u32() {
    if (n - pos < 4) { ok = false; return 0; }
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(p[pos + i]) << (8 * i);
    pos += 4;
    return v;
  }
  uint64_t u64() {
    if (n - pos < 8) { ok = false; return 0; }
    uint64_t v = 0;
    for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(p[pos + i]) << (8 * i);
    pos += 8;
    return v;
  }
  std::string str(uint64_t len) {
    if (len > n - pos) { ok = false; return {}; }  // subtraction form: a huge length cannot wrap
    std::string s(reinterpret_cast<const char*>(p + pos), static_cast<size_t>(len));
    pos += static_cast<size_t>(len);
    return s;
  }
};

const int kDtypeSize[8] = {4, 8, 2, 2, 4, 8, 1, 1};

}  // namespace

// Writes `n` tensors.  dims_flat holds the dims of all tensors back to back.
FB_API int fb_ser_save(const char* path, int n, const char* const* names, const int* ndims,
                       const long long* dims_flat, const int* dtypes, const void* const* data,
                       const unsigned long long* nbytes, char* err, int errlen) {
  std::vector<uint8_t> header;
  uint64_t data_size = 0;
  for (int i = 0; i < n; ++i) data_size += nbytes[i];
  put_u32(header, 1);
  put_u64(header, static_cast<uint64_t>(n));
  put_u64(header, data_size);
  put_u64(header, static_cast<uint64_t>(n));
  uint64_t offset = 0;
  size_t dpos = 0;
  for (int i = 0; i < n; ++i) {
    if (dtypes[i] < 0 || dtypes[i] > 7) {
      set_err(err, errlen, "unknown dtype code for tensor '" + std::string(names[i]) + "'");
      return -1;
    }
    uint64_t numel = 1;
    for (int d = 0; d < ndims[i]; ++d) numel *= static_cast<uint64_t>(dims_flat[dpos + d]);
    if (numel * kDtypeSize[dtypes[i]] != nbytes[i]) {
      set_err(err, errlen, "byte size does not match shape for tensor '" + std::string(names[i]) + "'");
      return -1;
    }
    const size_t len = std::strlen(names[i]);
    put_u64(header, len);
    header.insert(header.end(), names[i], names[i] + len);
    put_u64(header, static_cast<uint64_t>(ndims[i]));
    for (int d = 0; d < ndims[i]; ++d) put_u64(header, static_cast<uint64_t>(dims_flat[dpos + d]));
    dpos += static_cast<size_t>(ndims[i]);
    put_u32(header, static_cast<uint32_t>(dtypes[i]));
    put_u64(header, offset);
    put_u64(header, nbytes[i]);
    offset += nbytes[i];
  }
  FILE* f = std::fopen(path, "wb");
  if (f == nullptr) {
    set_err(err, errlen, std::string("Failed to create file: ") + path);
    return -2;
  }
  bool ok = std::fwrite("FERRUM01", 1, 8, f) == 8;
  std::vector<uint8_t> len8;
  put_u64(len8, header.size());
  ok = ok && std::fwrite(len8.data(), 1, 8, f) == 8;
  ok = ok && std::fwrite(header.data(), 1, header.size(), f) == header.size();
  for (int i = 0; ok && i < n; ++i) {
    if (nbytes[i] > 0) ok = std::fwrite(data[i], 1, nbytes[i], f) == nbytes[i];
  }
  ok = (std::fflush(f) == 0) && ok;
  std::fclose(f);
  if (!ok) {
    set_err(err, errlen, std::string("Failed to write file: ") + path);
    return -3;
  }
  return 0;
}

namespace {
void* open_impl(const char* path, char* err, int errlen) {
  FILE* f = std::fopen(path, "rb");
  if (f == nullptr) {
    set_err(err, errlen, std::string("Failed to open file: ") + path);
    return nullptr;
  }
  uint8_t head[16];
  if (std::fread(head, 1, 16, f) != 16) {
    std::fclose(f);
    set_err(err, errlen, "Failed to read magic: file too short");
    return nullptr;
  }
  if (std::memcmp(head, "FERRUM01", 8) != 0) {
    std::fclose(f);
    set_err(err, errlen, "Invalid file format: bad magic bytes");
    return nullptr;
  }
  uint64_t hlen = 0;
  for (int i = 0; i < 8; ++i) hlen |= static_cast<uint64_t>(head[8 + i]) << (8 * i);
  std::fseek(f, 0, SEEK_END);
  const long fsize = std::ftell(f);
  if (hlen > static_cast<uint64_t>(fsize) || hlen < 28) {
    std::fclose(f);
    set_err(err, errlen, "Failed to read header: implausible header length");
    return nullptr;
  }
  std::fseek(f, 16, SEEK_SET);
  std::vector<uint8_t> hb(static_cast<size_t>(hlen));
  if (std::fread(hb.data(), 1, hb.size(), f) != hb.size()) {
    std::fclose(f);
    set_err(err, errlen, "Failed to read header");
    return nullptr;
  }
  Cursor c{hb.data(), hb.size()};
  Reader* r = new Reader();
  r->f = f;
  r->version = c.u32();
  const uint64_t num = c.u64();
  r->data_size = c.u64();
  const uint64_t map_len = c.u64();
  (void)num;
  // an entry takes at least 36 header bytes (name length, rank, dtype, offset, size), so a count the header
  // cannot hold is rejected before anything is reserved for it
  if (map_len > hlen / 36) c.ok = false;
  for (uint64_t i = 0; c.ok && i < map_len; ++i) {
    Entry e;
    e.name = c.str(c.u64());
    const uint64_t nd = c.u64();
    if (nd > 64) { c.ok = false; break; }
    for (uint64_t d = 0; d < nd; ++d) e.dims.push_back(c.u64());
    e.dtype = c.u32();
    e.offset = c.u64();
    e.size = c.u64();
    if (e.dtype > 7 || e.size > r->data_size || e.offset > r->data_size - e.size) c.ok = false;
    r->entries.push_back(std::move(e));
  }
  if (!c.ok) {
    std::fclose(f);
    delete r;
    set_err(err, errlen, "Failed to deserialize header");
    return nullptr;
  }
  r->data_start = 16 + hlen;
  if (r->data_start > static_cast<uint64_t>(fsize) || r->data_size > static_cast<uint64_t>(fsize) - r->data_start) {
    std::fclose(f);
    delete r;
    set_err(err, errlen, "Failed to read data: file is truncated");
    return nullptr;
  }
  return r;
}
}  // namespace

// No C++ exception crosses the C boundary: an allocation failure while parsing a hostile header becomes an error
// string like every other defect of the file.
FB_API void* fb_ser_open(const char* path, char* err, int errlen) {
  try {
    return open_impl(path, err, errlen);
  } catch (const std::exception& e) {
    set_err(err, errlen, std::string("Failed to deserialize header: ") + e.what());
    return nullptr;
  }
}

FB_API int fb_ser_count(void* h) { return static_cast<int>(static_cast<Reader*>(h)->entries.size()); }
FB_API unsigned int fb_ser_version(void* h) { return static_cast<Reader*>(h)->version; }

FB_API int fb_ser_meta(void* h, int i, char* name_buf, int name_cap, int* ndim, long long* dims, int dims_cap,
                       int* dtype, unsigned long long* offset, unsigned long long* size) {
  Reader* r = static_cast<Reader*>(h);
  if (i < 0 || i >= static_cast<int>(r->entries.size())) return -1;
  const Entry& e = r->entries[static_cast<size_t>(i)];
  if (static_cast<int>(e.name.size()) + 1 > name_cap || static_cast<int>(e.dims.size()) > dims_cap) return -2;
  std::memcpy(name_buf, e.name.c_str(), e.name.size() + 1);
  *ndim = static_cast<int>(e.dims.size());
  for (size_t d = 0; d < e.dims.size(); ++d) dims[d] = static_cast<long long>(e.dims[d]);
  *dtype = static_cast<int>(e.dtype);
  *offset = e.offset;
  *size = e.size;
  return 0;
}
FB_API int fb_ser_name_len(void* h, int i) {
  Reader* r = static_cast<Reader*>(h);
  if (i < 0 || i >= static_cast<int>(r->entries.size())) return -1;
  return static_cast<int>(r->entries[static_cast<size_t>(i)].name.size());
}

FB_API int fb_ser_read(void* h, int i, void* dst) {
  Reader* r = static_cast<Reader*>(h);
  if (i < 0 || i >= static_cast<int>(r->entries.size())) return -1;
  const Entry& e = r->entries[static_cast<size_t>(i)];
  if (e.size == 0) return 0;
  if (std::fseek(r->f, static_cast<long>(r->data_start + e.offset), SEEK_SET) != 0) return -2;
  return std::fread(dst, 1, e.size, r->f) == e.size ? 0 : -3;
}

FB_API void fb_ser_close(void* h) {
  Reader* r = static_cast<Reader*>(h);
  if (r == nullptr) return;
  if (r->f) std::fclose(r->f);
  delete r;
}
