// Stand-in for the header protoc would generate from apache/singa's
// src/proto/core.proto (:22-78): the three enums, their *_Name helpers and the
// two messages the core library touches, written by hand because protoc is
// not available where the comparator is built.  TEST INFRASTRUCTURE ONLY: it
// lets the reference's own tensor / device sources compile unmodified into
// oracle/_ref/ (see oracle/ref_core_build.py).  Serialisation to the wire
// format is not provided (nothing on the compared path uses it).
#ifndef SINGA_PROTO_CORE_PB_H_
#define SINGA_PROTO_CORE_PB_H_
#include <cstdint>
#include <string>
#include <vector>

namespace singa {

enum DataType { kFloat32 = 0, kFloat16 = 1, kInt = 2, kChar = 3, kDouble = 4, kUChar = 5, kNumDataType = 6 };
enum LangType { kCpp = 0, kCuda = 1, kOpencl = 2, kNumDeviceType = 4 };
enum CopyDirection {
  kHostToHost = 0,
  kHostToDevice = 1,
  kDeviceToHost = 2,
  kDeviceToDevice = 3,
  kNumDirection = 4
};

inline const std::string& DataType_Name(DataType v) {
  static const std::string names[] = {"kFloat32", "kFloat16", "kInt", "kChar", "kDouble", "kUChar", "kNumDataType"};
  static const std::string unknown = "unknown";
  return v >= 0 && v <= kNumDataType ? names[v] : unknown;
}
inline const std::string& LangType_Name(LangType v) {
  static const std::string names[] = {"kCpp", "kCuda", "kOpencl", "unknown", "kNumDeviceType"};
  static const std::string unknown = "unknown";
  return v >= 0 && v <= kNumDeviceType ? names[v] : unknown;
}

class MemPoolConf {
 public:
  const std::string& type() const { return type_; }
  void set_type(const std::string& v) { type_ = v; }
  uint32_t init_size() const { return init_size_; }
  void set_init_size(uint32_t v) { init_size_ = v; }
  uint32_t max_size() const { return max_size_; }
  void set_max_size(uint32_t v) { max_size_ = v; }
  uint32_t flag() const { return flag_; }
  void set_flag(uint32_t v) { flag_ = v; }
  const std::vector<uint32_t>& device() const { return device_; }
  uint32_t device(int i) const { return device_[i]; }
  int device_size() const { return static_cast<int>(device_.size()); }
  void add_device(uint32_t v) { device_.push_back(v); }
  void clear_device() { device_.clear(); }

 private:
  std::string type_ = "cnmem";
  uint32_t init_size_ = 256, max_size_ = 0, flag_ = 0;
  std::vector<uint32_t> device_;
};

class TensorProto {
 public:
  const std::vector<uint32_t>& shape() const { return shape_; }
  void add_shape(uint32_t v) { shape_.push_back(v); }
  void clear_shape() { shape_.clear(); }
  DataType data_type() const { return data_type_; }
  void set_data_type(DataType v) { data_type_ = v; }
  const std::vector<int32_t>& stride() const { return stride_; }
  void add_stride(int32_t v) { stride_.push_back(v); }
  void clear_stride() { stride_.clear(); }
  float float_data(int i) const { return float_data_[i]; }
  void add_float_data(float v) { float_data_.push_back(v); }
  void clear_float_data() { float_data_.clear(); }
  int float_data_size() const { return static_cast<int>(float_data_.size()); }
  double double_data(int i) const { return double_data_[i]; }
  void add_double_data(double v) { double_data_.push_back(v); }
  void clear_double_data() { double_data_.clear(); }
  int32_t int_data(int i) const { return int_data_[i]; }
  void add_int_data(int32_t v) { int_data_.push_back(v); }
  void clear_int_data() { int_data_.clear(); }
  unsigned char bytes_data(size_t i) const { return bytes_data_[i]; }
  void add_bytes_data(unsigned char v) { bytes_data_.push_back(v); }
  void clear_bytes_data() { bytes_data_.clear(); }

 private:
  std::vector<uint32_t> shape_;
  DataType data_type_ = kFloat32;
  std::vector<int32_t> stride_;
  std::vector<float> float_data_;
  std::vector<double> double_data_;
  std::vector<int32_t> int_data_;
  std::vector<unsigned char> bytes_data_;
};

}  // namespace singa
#endif  // SINGA_PROTO_CORE_PB_H_
