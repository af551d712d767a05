// Protocol-buffers wire format, just enough of it to read and write the reference's cache files
// (tc/proto/compcache.proto, tc/proto/mapping_options.proto: proto2, scalar fields are varints,
// strings and sub-messages are length-delimited, repeated scalars are not packed).  The files stay
// interchangeable with ones written by the reference's generated protobuf classes; no protobuf
// library is needed to build or run.
#pragma once

#include <cstdint>
#include <string>

namespace tc {
namespace proto {

enum WireType : uint32_t { kVarint = 0, kFixed64 = 1, kBytes = 2, kFixed32 = 5 };

class Writer {
 public:
  void varint(uint32_t field, uint64_t value) {
    raw((uint64_t)field << 3 | kVarint);
    raw(value);
  }
  void boolean(uint32_t field, bool value) { varint(field, value ? 1 : 0); }
  void bytes(uint32_t field, const std::string& value) {
    raw((uint64_t)field << 3 | kBytes);
    raw(value.size());
    out_ += value;
  }
  void message(uint32_t field, const Writer& sub) { bytes(field, sub.out_); }
  const std::string& str() const { return out_; }

 private:
  void raw(uint64_t v) {
    while (v >= 0x80) {
      out_.push_back((char)(v | 0x80));
      v >>= 7;
    }
    out_.push_back((char)v);
  }
  std::string out_;
};

// Walks the fields of one message.  next() returns false at the end of the buffer or on malformed
// input (ok() tells which); unknown fields can simply be ignored by the caller.
class Reader {
 public:
  Reader(const char* data, size_t size) : p_(data), end_(data + size) {}
  explicit Reader(const std::string& s) : Reader(s.data(), s.size()) {}

  bool next() {
    if (p_ == end_ || !ok_) return false;
    uint64_t key;
    if (!raw(&key)) return fail();
    field_ = (uint32_t)(key >> 3);
    type_ = (uint32_t)(key & 7);
    switch (type_) {
      case kVarint:
        return raw(&value_) || fail();
      case kFixed64:
        return fixed(8) || fail();
      case kFixed32:
        return fixed(4) || fail();
      case kBytes: {
        uint64_t n;
        if (!raw(&n) || n > (uint64_t)(end_ - p_)) return fail();
        bytes_ = p_;
        size_ = (size_t)n;
        p_ += n;
        return true;
      }
      default:
        return fail();  // groups are not used by these messages
    }
  }
  bool ok() const { return ok_; }
  uint32_t field() const { return field_; }
  bool isVarint() const { return type_ == kVarint; }
  bool isBytes() const { return type_ == kBytes; }
  uint64_t value() const { return value_; }
  std::string string() const { return std::string(bytes_, size_); }
  Reader sub() const { return Reader(bytes_, size_); }
  // One element of a packed repeated scalar (the buffer is a run of bare varints): false at the end.
  bool packed(uint64_t* v) { return p_ != end_ && (raw(v) || fail()); }
  // A repeated uint64 field arrives either as one varint per element or as a packed run; a proto2
  // parser has to take both.  Appends the element(s) of the current field.
  template <typename Vec>
  void appendTo(Vec* out) const {
    if (isVarint()) {
      out->push_back((typename Vec::value_type)value_);
    } else if (isBytes()) {
      Reader run = sub();
      uint64_t v;
      while (run.packed(&v)) out->push_back((typename Vec::value_type)v);
    }
  }

 private:
  bool fail() {
    ok_ = false;
    return false;
  }
  bool raw(uint64_t* v) {
    uint64_t r = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (p_ == end_) return false;
      const uint8_t b = (uint8_t)*p_++;
      r |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) {
        *v = r;
        return true;
      }
    }
    return false;
  }
  bool fixed(int n) {
    if (end_ - p_ < n) return false;
    value_ = 0;
    for (int i = 0; i < n; ++i) value_ |= (uint64_t)(uint8_t)p_[i] << (8 * i);
    p_ += n;
    return true;
  }
  const char* p_;
  const char* end_;
  bool ok_ = true;
  uint32_t field_ = 0, type_ = 0;
  uint64_t value_ = 0;
  const char* bytes_ = nullptr;
  size_t size_ = 0;
};

}  // namespace proto
}  // namespace tc
