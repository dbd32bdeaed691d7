#include "npz.h"

#include <zlib.h>

#include <cstring>
#include <fstream>

namespace turbo_transformers {
namespace loaders {

namespace {

uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint64_t rd64(const uint8_t* p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

constexpr uint32_t kEocd = 0x06054b50, kEocd64 = 0x06064b50, kEocd64Loc = 0x07064b50, kCentral = 0x02014b50, kLocal = 0x04034b50;

// The zip64 extended-information extra field (id 1) carries, in this order, only those of {uncompressed size, compressed
// size, local header offset} whose 32-bit field holds 0xFFFFFFFF.
void apply_zip64_extra(const uint8_t* extra, size_t len, uint64_t* usize, uint64_t* csize, uint64_t* offset) {
  size_t pos = 0;
  while (pos + 4 <= len) {
    const uint16_t id = rd16(extra + pos), sz = rd16(extra + pos + 2);
    const uint8_t* f = extra + pos + 4;
    if (id == 1) {
      size_t q = 0;
      if (usize && *usize == 0xFFFFFFFFu && q + 8 <= sz) { *usize = rd64(f + q); q += 8; }
      if (csize && *csize == 0xFFFFFFFFu && q + 8 <= sz) { *csize = rd64(f + q); q += 8; }
      if (offset && *offset == 0xFFFFFFFFu && q + 8 <= sz) { *offset = rd64(f + q); q += 8; }
      return;
    }
    pos += 4 + (size_t)sz;
  }
}

std::string dict_value(const std::string& header, const std::string& key) {
  const size_t k = header.find("'" + key + "'");
  TT_ENFORCE(k != std::string::npos, "npy header has no '%s'", key.c_str());
  size_t c = header.find(':', k);
  TT_ENFORCE(c != std::string::npos, "npy header: no value for '%s'", key.c_str());
  ++c;
  while (c < header.size() && header[c] == ' ') ++c;
  size_t e = c;
  if (header[c] == '(') {
    e = header.find(')', c);
    TT_ENFORCE(e != std::string::npos, "npy header: unterminated shape");
    return header.substr(c, e - c + 1);
  }
  while (e < header.size() && header[e] != ',' && header[e] != '}') ++e;
  return header.substr(c, e - c);
}

}  // namespace

size_t NpyArray::num_vals() const {
  size_t n = 1;
  for (int64_t d : shape) n *= (size_t)d;
  return n;
}

NpyArray npy_parse(const uint8_t* data, size_t size, const std::string& what) {
  TT_ENFORCE(size >= 10 && std::memcmp(data, "\x93NUMPY", 6) == 0, "%s is not an npy image", what.c_str());
  const int major = data[6];
  size_t hlen, hoff;
  if (major == 1) {
    hlen = rd16(data + 8);
    hoff = 10;
  } else {
    TT_ENFORCE(size >= 12, "%s: truncated npy header", what.c_str());
    hlen = rd32(data + 8);
    hoff = 12;
  }
  TT_ENFORCE(hoff + hlen <= size, "%s: truncated npy header", what.c_str());
  const std::string header(reinterpret_cast<const char*>(data + hoff), hlen);
  NpyArray a;
  std::string descr = dict_value(header, "descr");
  TT_ENFORCE(descr.size() >= 2 && (descr[0] == '\'' || descr[0] == '"'), "%s: structured dtypes are not supported", what.c_str());
  a.descr = descr.substr(1, descr.find(descr[0], 1) - 1);
  a.fortran_order = dict_value(header, "fortran_order").rfind("True", 0) == 0;
  const std::string shape = dict_value(header, "shape");
  for (size_t i = 1; i < shape.size();) {
    while (i < shape.size() && (shape[i] == ' ' || shape[i] == ',')) ++i;
    if (i >= shape.size() || shape[i] == ')') break;
    size_t j = i;
    while (j < shape.size() && shape[j] >= '0' && shape[j] <= '9') ++j;
    TT_ENFORCE(j > i, "%s: bad shape '%s'", what.c_str(), shape.c_str());
    a.shape.push_back(std::stoll(shape.substr(i, j - i)));
    i = j;
  }
  TT_ENFORCE(a.descr.size() >= 3 && (a.descr[0] == '<' || a.descr[0] == '|' || a.descr[0] == '='),
             "%s: dtype '%s' is not little-endian", what.c_str(), a.descr.c_str());
  a.word_size = (size_t)std::stoul(a.descr.substr(2));
  TT_ENFORCE(!a.fortran_order || a.shape.size() <= 1, "%s: Fortran-ordered arrays are not supported", what.c_str());
  const size_t nbytes = a.num_vals() * a.word_size;
  TT_ENFORCE(hoff + hlen + nbytes <= size, "%s: payload shorter than its shape says", what.c_str());
  a.bytes.assign(data + hoff + hlen, data + hoff + hlen + nbytes);
  return a;
}

npz_t npz_load(const std::string& filename) {
  std::ifstream f(filename, std::ios::binary | std::ios::ate);
  TT_ENFORCE(f.good(), "cannot open %s", filename.c_str());
  const size_t size = (size_t)f.tellg();
  std::vector<uint8_t> buf(size);
  f.seekg(0);
  f.read(reinterpret_cast<char*>(buf.data()), (std::streamsize)size);
  TT_ENFORCE(f.good() && size >= 22, "%s is not a zip archive", filename.c_str());
  // end-of-central-directory record: the last one in the file (the trailing comment is at most 65535 bytes)
  size_t eocd = size;
  for (size_t i = size - 22, stop = size > 22 + 65535 ? size - 22 - 65535 : 0;; --i) {
    if (rd32(&buf[i]) == kEocd) {
      eocd = i;
      break;
    }
    if (i == stop) break;
  }
  TT_ENFORCE(eocd != size, "%s: no zip end-of-central-directory record", filename.c_str());
  uint64_t entries = rd16(&buf[eocd + 10]), cd_off = rd32(&buf[eocd + 16]);
  if ((entries == 0xFFFF || cd_off == 0xFFFFFFFFu) && eocd >= 20 && rd32(&buf[eocd - 20]) == kEocd64Loc) {
    const uint64_t e64 = rd64(&buf[eocd - 20 + 8]);
    TT_ENFORCE(e64 + 56 <= size && rd32(&buf[e64]) == kEocd64, "%s: bad zip64 end record", filename.c_str());
    entries = rd64(&buf[e64 + 32]);
    cd_off = rd64(&buf[e64 + 48]);
  }
  npz_t out;
  size_t pos = (size_t)cd_off;
  for (uint64_t e = 0; e < entries; ++e) {
    TT_ENFORCE(pos + 46 <= size && rd32(&buf[pos]) == kCentral, "%s: bad central directory entry %llu", filename.c_str(), (unsigned long long)e);
    const uint16_t method = rd16(&buf[pos + 10]);
    uint64_t csize = rd32(&buf[pos + 20]), usize = rd32(&buf[pos + 24]), lho = rd32(&buf[pos + 42]);
    const uint16_t nlen = rd16(&buf[pos + 28]), xlen = rd16(&buf[pos + 30]), clen = rd16(&buf[pos + 32]);
    TT_ENFORCE(pos + 46 + nlen + xlen + clen <= size, "%s: truncated central directory", filename.c_str());
    std::string name(reinterpret_cast<const char*>(&buf[pos + 46]), nlen);
    apply_zip64_extra(&buf[pos + 46 + nlen], xlen, &usize, &csize, &lho);
    pos += 46 + (size_t)nlen + xlen + clen;
    TT_ENFORCE(lho + 30 <= size && rd32(&buf[lho]) == kLocal, "%s: bad local header of %s", filename.c_str(), name.c_str());
    const size_t data_off = (size_t)lho + 30 + rd16(&buf[lho + 26]) + rd16(&buf[lho + 28]);
    TT_ENFORCE(data_off + csize <= size, "%s: member %s runs past the end of the file", filename.c_str(), name.c_str());
    if (name.size() > 4 && name.compare(name.size() - 4, 4, ".npy") == 0) name.resize(name.size() - 4);
    if (method == 0) {
      out.emplace(name, npy_parse(&buf[data_off], (size_t)csize, name));
    } else {
      TT_ENFORCE(method == 8, "%s: member %s uses zip method %d (only stored and deflate are supported)", filename.c_str(), name.c_str(),
                 (int)method);
      std::vector<uint8_t> raw((size_t)usize);
      z_stream zs;
      std::memset(&zs, 0, sizeof(zs));
      TT_ENFORCE(inflateInit2(&zs, -MAX_WBITS) == Z_OK, "zlib inflateInit2 failed");
      zs.next_in = &buf[data_off];
      zs.avail_in = (uInt)csize;
      zs.next_out = raw.data();
      zs.avail_out = (uInt)usize;
      TT_ENFORCE(csize < (1ull << 32) && usize < (1ull << 32), "%s: member %s is too large for one inflate call", filename.c_str(), name.c_str());
      const int rc = inflate(&zs, Z_FINISH);
      inflateEnd(&zs);
      TT_ENFORCE(rc == Z_STREAM_END && zs.total_out == usize, "%s: member %s does not inflate to its stated size", filename.c_str(), name.c_str());
      out.emplace(name, npy_parse(raw.data(), raw.size(), name));
    }
  }
  return out;
}

NpyArray& NPZMapView::operator[](const std::string& key) {
  const std::string actual = prefix_ + key;
  auto it = npz_->find(actual);
  TT_ENFORCE(it != npz_->end(), "cannot find parameter %s in npz file", actual.c_str());
  return it->second;
}

bool NPZMapView::IsExist(const std::string& subprefix) const {
  const std::string actual = prefix_ + subprefix;
  auto it = npz_->lower_bound(actual);
  return it != npz_->end() && it->first.compare(0, actual.size(), actual) == 0;
}

core::Tensor NPZLoader::LoadFloat(const std::string& name) {
  NpyArray& a = view_[name];
  TT_ENFORCE(device_ == kDLCUDA, "NPZLoader places tensors on a CUDA device (there is no CPU path)");
  TT_ENFORCE(a.descr == "<f4" || a.descr == "<f2", "parameter %s has dtype %s; float32 or float16 expected", name.c_str(), a.descr.c_str());
  const int src = a.descr == "<f4" ? TTB_F32 : TTB_F16;
  const int dst = core::ToTTBDtype(dtype_);
  ttb_ctx* c = core::DeviceContext(device_id_);
  core::Tensor t(nullptr);
  t.Reshape(dtype_, a.shape, kDLCUDA, device_id_, "NPZLoader/" + name);
  const int64_t n = (int64_t)a.num_vals();
  if (n == 0) return t;
  if (src == dst) {
    TT_ENFORCE(ttb_memcpy_h2d(c, t.raw_mut(), a.bytes.data(), a.bytes.size()) == TTB_OK, "upload of %s failed: %s", name.c_str(), ttb_last_error(c));
  } else {
    // upload as stored, convert on the device (the re-layout entry point with an [N,K] source only converts)
    core::Tensor staged(nullptr);
    staged.Reshape(src == TTB_F32 ? DLDataType{kDLFloat, 32, 1} : DLDataType{kDLFloat, 16, 1}, a.shape, kDLCUDA, device_id_, "NPZLoader/staging");
    TT_ENFORCE(ttb_memcpy_h2d(c, staged.raw_mut(), a.bytes.data(), a.bytes.size()) == TTB_OK, "upload of %s failed: %s", name.c_str(), ttb_last_error(c));
    TT_ENFORCE(ttb_prepack_weight(c, src, staged.raw(), 1, n, 1, dst, t.raw_mut()) == TTB_OK, "conversion of %s failed: %s", name.c_str(),
               ttb_last_error(c));
    TT_ENFORCE(ttb_ctx_sync(c) == TTB_OK, "sync failed");  // `staged` is released when this returns
  }
  return t;
}

}  // namespace loaders
}  // namespace turbo_transformers
