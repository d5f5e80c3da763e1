// TEST INFRASTRUCTURE ONLY - never linked into, imported by or called from the product path.
//
// C-ABI shim over the reference's own host functions, so that the checker can call the
// UNMODIFIED reference sources (compiled where they lie, see build_ref.py) through ctypes.
// The three functions wrapped here are the reference's
//   weight_prepacking_fp16_to_fp6   (fp6_marlin/weight_quant.cpp:106-124)
//   weight_matrix_prepacking        (fp6_marlin/weight_prepacking.cpp:123-177)
//   dequantMatrix_fp6_to_fp16       (fp6_marlin/weight_prepacking.cpp:180-217)
// and the argument order below follows what fp6_marlin/pybind.cpp:18-87 passes them.
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <cuda_fp16.h>

void weight_prepacking_fp16_to_fp6(uint16_t* weight_16bit, uint8_t* weight_6bit_packed, size_t K, size_t N);
void weight_matrix_prepacking(int* packed_weights, int* FP6Weights, size_t K, size_t N);
void dequantMatrix_fp6_to_fp16(half* A_16bit_h, unsigned char* A_x_bit_h, size_t M, size_t K, half* scale);

extern "C" {

// rows x cols fp16 (row-major memory, packed as it lies) -> rows*cols*6/8 bytes.
// Returns 0, or 1 when the reference throws std::invalid_argument (value out of FP6 range).
int ref_quantize_fp6(const uint16_t* w, uint8_t* out, size_t rows, size_t cols) {
  try {
    weight_prepacking_fp16_to_fp6(const_cast<uint16_t*>(w), out, rows, cols);
  } catch (const std::invalid_argument&) {
    return 1;
  }
  return 0;
}

// fp6 stream viewed as (n rows, k cols) -> the reference "2+4" tensor-core layout, same byte count.
int ref_prepack_fp6(const uint8_t* fp6, uint8_t* out, size_t n, size_t k) {
  weight_matrix_prepacking(reinterpret_cast<int*>(out),
                           reinterpret_cast<int*>(const_cast<uint8_t*>(fp6)), n, k);
  return 0;
}

// fp6 stream (n rows, k cols) + per-row fp16 scale -> (n, k) fp16.
int ref_dequant_fp6(const uint8_t* fp6, const uint16_t* scale, uint16_t* out, size_t n, size_t k) {
  dequantMatrix_fp6_to_fp16(reinterpret_cast<half*>(out), const_cast<uint8_t*>(fp6), n, k,
                            reinterpret_cast<half*>(const_cast<uint16_t*>(scale)));
  return 0;
}

}  // extern "C"
