/*
 * DECX.h -- the part of DECX's public C++ interface that lies on the dense-contraction path
 * (fp32 GEMM and im2col convolution), implemented over the C ABI of include/decxb.h.
 *
 * Same names, argument meaning and error behaviour as the reference's headers (its own
 * umbrella header APIs/DECX.h is missing from its repository; the declarations below follow
 * the class and function headers, cited per item, paths relative to the reference root):
 * abstract container classes created through factory functions, operations as free functions
 * in de::cuda taking abstract references and returning a de::DH handle by value.  float
 * instantiations only.  Link with -ldecx_b200 -ldecxb.
 */
#ifndef DECX_B200_DECX_H_
#define DECX_B200_DECX_H_

#include <cstddef>

typedef unsigned int uint;

namespace decx {
/* srcs/handles/decx_handles.h:6-38 */
enum DECX_error_types {
    DECX_SUCCESS = 0x00, DECX_FAIL_not_init = 0x01, DECX_FAIL_DimsNotMatching = 0x03, DECX_FAIL_ConvBadKernel = 0x05,
    DECX_FAIL_ErrorFlag = 0x0b, DECX_FAIL_ErrorParams = 0x0d, DECX_FAIL_MNumNotMatching = 0x0f, DECX_FAIL_ALLOCATION = 0x10
};
/* srcs/classes/store_types.h:24-28 */
enum DATA_STORE_TYPE { Page_Locked = 0x00, Page_Default = 0x01 };
/* srcs/convolution/CUDA/conv_flags.h:16-20 */
enum conv_property { de_conv_no_compensate = 0, de_conv_zero_compensate = 1 };
}  // namespace decx

namespace de {

/* srcs/handles/decx_handles.h:44-48: error_string points at a static literal. */
typedef struct DECX_Handle {
    int error_type;
    char* error_string;
} DH;

/* srcs/classes/classes_util.h:59-62: storage type of IEEE half values. */
struct alignas(2) Half { unsigned short val; };

/* srcs/core/configs/config.h:62-78.  Must be called before any de::cuda operation;
 * operations return DECX_FAIL_not_init otherwise (srcs/GEMM/CUDA/large_squares/GEMM.h:63-66). */
void InitCuda();
/* srcs/core/memory_management/Memory_pool.h:28-38 */
void release_all_tmp();

/* ---- srcs/classes/Matrix.h:34-65: row-major, pitch = ceil8(width) floats (:253-267) ------- */
template <typename T>
class Matrix {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual size_t TotalBytes() = 0;
    virtual T& index(const int row, const int col) = 0;
    virtual void release() = 0;
    virtual Matrix<T>& operator=(Matrix<T>& src) = 0;   /* aliases the storage (ref-counted), Matrix.h:509-530 */
    virtual ~Matrix() {}
};
template <typename T> Matrix<T>& CreateMatrixRef();
template <typename T> Matrix<T>* CreateMatrixPtr();
template <typename T> Matrix<T>& CreateMatrixRef(const uint width, const uint height, const int store_type);
template <typename T> Matrix<T>* CreateMatrixPtr(const uint width, const uint height, const int store_type);

/* ---- srcs/classes/MatrixArray.h:27-53: MatrixNum matrices of one size, contiguous,
 *      pitch*height floats apart (:222-237); index(row, col, matrix) (:367-370) ----------------- */
template <typename T>
class MatrixArray {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual uint MatrixNumber() = 0;
    virtual T& index(uint row, uint col, size_t _seq) = 0;
    virtual MatrixArray<T>& operator=(MatrixArray<T>& src) = 0;
    virtual void release() = 0;
    virtual ~MatrixArray() {}
};
template <typename T> MatrixArray<T>& CreateMatrixArrayRef();
template <typename T> MatrixArray<T>* CreateMatrixArrayPtr();
template <typename T> MatrixArray<T>& CreateMatrixArrayRef(uint width, uint height, uint MatrixNum, const int flag);
template <typename T> MatrixArray<T>* CreateMatrixArrayPtr(uint width, uint height, uint MatrixNum, const int flag);

/* ---- srcs/classes/GPU_Matrix.h:21-50 ---------------------------------------------------------- */
template <typename T>
class GPU_Matrix {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual size_t TotalBytes() = 0;
    virtual void Load_from_host(Matrix<T>& src) = 0;
    virtual void Load_to_host(Matrix<T>& dst) = 0;
    virtual void release() = 0;
    virtual GPU_Matrix<T>& operator=(GPU_Matrix<T>& src) = 0;
    virtual ~GPU_Matrix() {}
};
template <typename T> GPU_Matrix<T>& CreateGPUMatrixRef();
template <typename T> GPU_Matrix<T>* CreateGPUMatrixPtr();
template <typename T> GPU_Matrix<T>& CreateGPUMatrixRef(const uint width, const uint height);
template <typename T> GPU_Matrix<T>* CreateGPUMatrixPtr(const uint width, const uint height);

/* ---- srcs/classes/Tensor.h:31-57: HWC, dpitch = ceil4(depth), wpitch = ceil4(width);
 *      index(x = row, y = column, z = channel) (:389-394); zero-filled on construction (:312) */
template <typename T>
class Tensor {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual uint Depth() = 0;
    virtual T& index(const int x, const int y, const int z) = 0;
    virtual Tensor<T>& operator=(Tensor<T>& src) = 0;
    virtual void release() = 0;
    virtual ~Tensor() {}
};
template <typename T> Tensor<T>& CreateTensorRef();
template <typename T> Tensor<T>* CreateTensorPtr();
template <typename T> Tensor<T>& CreateTensorRef(const uint width, const uint height, const uint depth, const int flag);
template <typename T> Tensor<T>* CreateTensorPtr(const uint width, const uint height, const uint depth, const int flag);

/* ---- srcs/classes/GPU_Tensor.h:22-51 ------------------------------------------------------------ */
template <typename T>
class GPU_Tensor {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual uint Depth() = 0;
    virtual GPU_Tensor<T>& operator=(GPU_Tensor<T>& src) = 0;
    virtual void Load_from_host(Tensor<T>& src) = 0;
    virtual void Load_to_host(Tensor<T>& dst) = 0;
    virtual void release() = 0;
    virtual ~GPU_Tensor() {}
};
template <typename T> GPU_Tensor<T>& CreateGPUTensorRef();
template <typename T> GPU_Tensor<T>* CreateGPUTensorPtr();
template <typename T> GPU_Tensor<T>& CreateGPUTensorRef(const uint width, const uint height, const uint depth);
template <typename T> GPU_Tensor<T>* CreateGPUTensorPtr(const uint width, const uint height, const uint depth);

/* ---- srcs/classes/TensorArray.h:24-53: tensors contiguous, dpitch*wpitch*height apart (:174-198) */
template <typename T>
class TensorArray {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual uint Depth() = 0;
    virtual uint TensorNum() = 0;
    virtual T& index(const int x, const int y, const int z, const int tensor_id) = 0;
    virtual TensorArray<T>& operator=(TensorArray<T>& src) = 0;
    virtual void release() = 0;
    virtual ~TensorArray() {}
};
template <typename T> TensorArray<T>& CreateTensorArrayRef();
template <typename T> TensorArray<T>* CreateTensorArrayPtr();
template <typename T> TensorArray<T>& CreateTensorArrayRef(const uint width, const uint height, const uint depth, const uint tensor_num, const int store_type);
template <typename T> TensorArray<T>* CreateTensorArrayPtr(const uint width, const uint height, const uint depth, const uint tensor_num, const int store_type);

/* ---- srcs/classes/GPU_TensorArray.h:23-55 -------------------------------------------------------- */
template <typename T>
class GPU_TensorArray {
public:
    virtual uint Width() = 0;
    virtual uint Height() = 0;
    virtual uint Depth() = 0;
    virtual uint TensorNum() = 0;
    virtual void Load_from_host(TensorArray<T>& src) = 0;
    virtual void Load_to_host(TensorArray<T>& dst) = 0;
    virtual GPU_TensorArray<T>& operator=(GPU_TensorArray<T>& src) = 0;
    virtual void release() = 0;
    virtual ~GPU_TensorArray() {}
};
template <typename T> GPU_TensorArray<T>& CreateGPUTensorArrayRef();
template <typename T> GPU_TensorArray<T>* CreateGPUTensorArrayPtr();
template <typename T> GPU_TensorArray<T>& CreateGPUTensorArrayRef(const uint width, const uint height, const uint depth, const uint tensor_num);
template <typename T> GPU_TensorArray<T>* CreateGPUTensorArrayPtr(const uint width, const uint height, const uint depth, const uint tensor_num);

namespace cuda {
/* srcs/GEMM/CUDA/large_squares/GEMM.h:27-31: dst = A*B and dst = A*B + C.  dst is
 * re-constructed to (B.width x A.height) by the callee (:73, :414). */
DH GEMM(Matrix<float>& A, Matrix<float>& B, Matrix<float>& dst);
DH GEMM(Matrix<float>& A, Matrix<float>& B, Matrix<float>& C, Matrix<float>& dst);
DH GEMM(GPU_Matrix<float>& A, GPU_Matrix<float>& B, GPU_Matrix<float>& dst);
DH GEMM(GPU_Matrix<float>& A, GPU_Matrix<float>& B, GPU_Matrix<float>& C, GPU_Matrix<float>& dst);

/* srcs/GEMM/CUDA/large_squares/GEMM.h:33-49: the same four entry points on half matrices
 * (pitch = ceil16(width) halves, Matrix.h:25,315).  Accumulation is fp32 here (the reference
 * accumulates in half). */
DH GEMM(Matrix<Half>& A, Matrix<Half>& B, Matrix<Half>& dst);
DH GEMM(Matrix<Half>& A, Matrix<Half>& B, Matrix<Half>& C, Matrix<Half>& dst);
DH GEMM(GPU_Matrix<Half>& A, GPU_Matrix<Half>& B, GPU_Matrix<Half>& dst);
DH GEMM(GPU_Matrix<Half>& A, GPU_Matrix<Half>& B, GPU_Matrix<Half>& C, GPU_Matrix<Half>& dst);

/* srcs/GEMM/CUDA/large_squares/GEMM3.h:27-37: dst[i] = A[i]*B[i] (+ C[i]) for every matrix of
 * the arrays, uploads, products and downloads overlapped. */
DH GEMM3(MatrixArray<float>& A, MatrixArray<float>& B, MatrixArray<float>& dst);
DH GEMM3(MatrixArray<float>& A, MatrixArray<float>& B, MatrixArray<float>& C, MatrixArray<float>& dst);

/* srcs/convolution/CUDA/im2col/conv2_mk_im2col.h:25: cross-correlation of src with every
 * tensor of `kernel`, stride 1; flag = decx::conv_property.  dst is re-constructed by the callee. */
DH Conv2_MK_im2col(Tensor<float>& src, TensorArray<float>& kernel, Tensor<float>& dst, const int flag);
/* Device-resident and batched forms (not in the reference, whose only entry is host-resident
 * and single-image): src/dst on the device; a TensorArray src convolves every image. */
DH Conv2_MK_im2col(GPU_Tensor<float>& src, GPU_TensorArray<float>& kernel, GPU_Tensor<float>& dst, const int flag);
DH Conv2_MK_im2col(GPU_TensorArray<float>& src, GPU_TensorArray<float>& kernel, GPU_TensorArray<float>& dst, const int flag);

/* Precision and algorithm switches of this implementation (no counterpart in the reference).
 * Default: 3xTF32 with K accumulated in chunks of 128 that are added in IEEE fp32 (within 1e-6 of
 * K max|a| max|b| also on same-sign data).  SetGemmStrictAccumulation(false) lets the tensor core
 * accumulate over all of K (a few percent faster; its round-toward-zero accumulator reaches
 * 2.9e-6 on the reference test program's all-positive matrices).  SetGemmPlainTF32(true) uses one
 * TF32 product instead of three.  SetConvExplicitPack(true): explicit pack + GEMM instead of the
 * default implicit convolution. */
void SetGemmPlainTF32(bool on);
void SetGemmStrictAccumulation(bool on);
void SetConvExplicitPack(bool on);
}  // namespace cuda
}  // namespace de

#endif
