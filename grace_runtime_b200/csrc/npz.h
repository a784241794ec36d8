// Reader for uncompressed .npz archives (ZIP "stored" members holding .npy arrays), the container of the
// kokkos.npz model format.  Arrays are converted by their stored dtype, never reinterpreted: the behaviour the
// reference loaders document in libgrace/src/npz3.h:105-149 (f4/f8/integers accepted for real arrays, integers and
// bools for index arrays, Fortran order rejected for arrays with more than one non-trivial dimension, non-finite
// values rejected).
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace gb {

struct ModelError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct NpyArray {
  char kind = 0;         // 'f', 'i', 'u', 'b', 'S'
  int word = 0;          // bytes per element
  bool fortran = false;
  std::vector<int64_t> shape;
  std::vector<unsigned char> data;
  int64_t size() const
  {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

class Npz {
 public:
  explicit Npz(const std::string &path);
  bool has(const std::string &key) const { return arrays_.count(key) != 0; }
  const NpyArray *find(const std::string &key) const;
  std::vector<std::string> keys() const;

  // real array as fp64 (empty when absent and !required)
  std::vector<double> reals(const std::string &key, bool required = true) const;
  // integer / bool array as int (empty when absent and !required)
  std::vector<int> ints(const std::string &key, bool required = true) const;
  double real_scalar(const std::string &key, double def) const;
  int int_scalar(const std::string &key, int def) const;
  int int_in(const std::string &key, int def, int lo, int hi) const;    // def outside [lo, hi]: the key is required
  std::vector<std::string> names(const std::string &key) const;
  std::vector<int64_t> shape(const std::string &key) const;
  void require_shape(const std::string &key, const std::vector<int64_t> &want) const;

 private:
  std::map<std::string, NpyArray> arrays_;
  std::string path_;
};

ModelError bad_array(const std::string &key, const std::string &what);

}    // namespace gb
