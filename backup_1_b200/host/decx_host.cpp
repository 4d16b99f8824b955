/*
 * The C++ de:: layer over the C ABI (include/decxb.h): container classes, factories, and the
 * de::cuda::GEMM / de::cuda::Conv2_MK_im2col entry points with the reference's conventions
 * (abstract references, dynamic_cast to the concrete class, callee re-constructs the result,
 * de::DH returned by value, blocking calls).  Pure host C++: every device action goes through
 * libdecxb.so.
 */
#include "decx/DECX.h"

#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>

#include "decxb.h"

namespace decx {

/* decx::cuP of the reference (srcs/core/configs/config.h:50): whether InitCuda ran. */
struct cudaProp { bool is_init = false; decxb_ctx* ctx = nullptr; bool plain_tf32 = false; bool strict = true; bool explicit_pack = false; };
static cudaProp cuP;

static inline uint ceil_to(uint v, uint m) { return (v + m - 1) / m * m; }

/* ---- handles (srcs/core/error.h:83-157) -------------------------------------------------------- */
static void set_handle(de::DH* h, int code, const char* text) { h->error_type = code; h->error_string = const_cast<char*>(text); }
static void Success(de::DH* h) { set_handle(h, DECX_SUCCESS, "No error"); }
static void Not_init(de::DH* h) { set_handle(h, DECX_FAIL_not_init, "CUDA should be initialized first"); }
static void MDim_Not_Matching(de::DH* h) { set_handle(h, DECX_FAIL_DimsNotMatching, "Matrix Dims don't match each other"); }
static void TDim_Not_Matching(de::DH* h) { set_handle(h, DECX_FAIL_DimsNotMatching, "Tensor Dims don't match each other"); }
static void from_status(de::DH* h, int rc)
{
    if (rc == DECXB_OK) { Success(h); return; }
    int code = rc;
    if (rc >= 100) code = rc == DECXB_ERR_NO_DEVICE || rc == DECXB_ERR_ARCH ? DECX_FAIL_not_init : DECX_FAIL_ErrorParams;
    set_handle(h, code, decxb_status_string(rc));
}

/* ---- storage: shared, so that operator= aliases like the reference's ref-counted pools --------- */
static std::shared_ptr<float> host_block(size_t bytes, int store_type)
{
    if (bytes == 0) return nullptr;
    float* p = nullptr;
    if (store_type == Page_Locked) {
        void* q = nullptr;
        if (decxb_host_alloc(bytes, &q) != DECXB_OK) throw std::bad_alloc();
        p = static_cast<float*>(q);
        memset(p, 0, bytes);
        return std::shared_ptr<float>(p, [](float* x) { decxb_host_free(x); });
    }
    void* q = nullptr;
    if (posix_memalign(&q, 64, (bytes + 63) / 64 * 64)) throw std::bad_alloc();
    memset(q, 0, bytes);
    return std::shared_ptr<float>(static_cast<float*>(q), [](float* x) { free(x); });
}

static std::shared_ptr<float> device_block(size_t bytes)
{
    if (bytes == 0) return nullptr;
    if (!cuP.ctx) throw std::runtime_error("de::InitCuda() must be called before GPU containers are created");
    void* q = nullptr;
    if (decxb_malloc(cuP.ctx, bytes, &q) != DECXB_OK) throw std::bad_alloc();
    decxb_memset(cuP.ctx, q, 0, bytes);
    decxb_ctx* ctx = cuP.ctx;
    return std::shared_ptr<float>(static_cast<float*>(q), [ctx](float* x) { decxb_free(ctx, x); });
}

/* ---- Matrix (float: pitch = ceil8(width); Half: pitch = ceil16(width), Matrix.h:24-25) ----------- */
template <typename T> struct mat_align { static constexpr uint value = 8; };
template <> struct mat_align<de::Half> { static constexpr uint value = 16; };

template <typename T>
class _MatrixT : public de::Matrix<T> {
public:
    uint width = 0, height = 0, pitch = 0;
    int Store_Type = Page_Default;
    size_t element_num = 0, total_bytes = 0, _element_num = 0, _total_bytes = 0;
    std::shared_ptr<float> Mat;                     /* raw storage; data() views it as T */

    T* data() { return reinterpret_cast<T*>(Mat.get()); }
    void _attribute_assign(uint w, uint h, int store)
    {
        width = w; height = h; Store_Type = store;
        pitch = ceil_to(w, mat_align<T>::value);
        element_num = (size_t)w * h; total_bytes = element_num * sizeof(T);
        _element_num = (size_t)pitch * h; _total_bytes = _element_num * sizeof(T);
    }
    void construct(uint w, uint h, int store) { _attribute_assign(w, h, store); Mat = host_block(_total_bytes, store); }
    void re_construct(uint w, uint h, int store)
    {
        if (w != width || h != height || store != Store_Type || !Mat) construct(w, h, store);   /* Matrix.h:239-248 */
    }
    _MatrixT() { _attribute_assign(0, 0, Page_Default); }
    _MatrixT(uint w, uint h, int store) { construct(w, h, store); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    size_t TotalBytes() override { return total_bytes; }
    T& index(const int row, const int col) override { return data()[(size_t)pitch * row + col]; }
    void release() override { Mat.reset(); }
    de::Matrix<T>& operator=(de::Matrix<T>& src) override
    {
        _MatrixT& s = dynamic_cast<_MatrixT&>(src);
        _attribute_assign(s.width, s.height, s.Store_Type);
        Mat = s.Mat;
        return *this;
    }
};
using _Matrix = _MatrixT<float>;
using _MatrixH = _MatrixT<de::Half>;

class _MatrixArray : public de::MatrixArray<float> {
public:
    uint width = 0, height = 0, pitch = 0;
    size_t ArrayNumber = 0, plane = 0, _plane = 0, total_bytes = 0;
    int _store_type = Page_Default;
    std::shared_ptr<float> MatArr;
    void _attribute_assign(uint w, uint h, uint n, int flag)
    {
        width = w; height = h; ArrayNumber = n; _store_type = flag;
        pitch = ceil_to(w, 8);                                      /* MatrixArray.h:230 */
        plane = (size_t)w * h; _plane = (size_t)pitch * h;
        total_bytes = _plane * n * sizeof(float);
    }
    void construct(uint w, uint h, uint n, int flag) { _attribute_assign(w, h, n, flag); MatArr = host_block(total_bytes, flag); }
    void re_construct(uint w, uint h, uint n, int flag)
    {
        if (w != width || h != height || n != ArrayNumber || flag != _store_type || !MatArr) construct(w, h, n, flag);
    }
    _MatrixArray() { _attribute_assign(0, 0, 0, Page_Default); }
    _MatrixArray(uint w, uint h, uint n, int flag) { construct(w, h, n, flag); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    uint MatrixNumber() override { return (uint)ArrayNumber; }
    float& index(uint row, uint col, size_t _seq) override { return MatArr.get()[_seq * _plane + (size_t)row * pitch + col]; }
    de::MatrixArray<float>& operator=(de::MatrixArray<float>& src) override
    {
        _MatrixArray& s = dynamic_cast<_MatrixArray&>(src);
        _attribute_assign(s.width, s.height, (uint)s.ArrayNumber, s._store_type);
        MatArr = s.MatArr;
        return *this;
    }
    void release() override { MatArr.reset(); }
};

template <typename T>
class _GPU_MatrixT : public de::GPU_Matrix<T> {
public:
    uint width = 0, height = 0, pitch = 0;
    size_t total_bytes = 0, _total_bytes = 0;
    std::shared_ptr<float> Mat;

    T* data() { return reinterpret_cast<T*>(Mat.get()); }
    void _attribute_assign(uint w, uint h)
    {
        width = w; height = h; pitch = ceil_to(w, mat_align<T>::value);   /* GPU_Matrix.h:211-223, :264 */
        total_bytes = (size_t)w * h * sizeof(T); _total_bytes = (size_t)pitch * h * sizeof(T);
    }
    void construct(uint w, uint h) { _attribute_assign(w, h); Mat = device_block(_total_bytes); }
    void re_construct(uint w, uint h) { if (w != width || h != height || !Mat) construct(w, h); }
    _GPU_MatrixT() { _attribute_assign(0, 0); }
    _GPU_MatrixT(uint w, uint h) { construct(w, h); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    size_t TotalBytes() override { return total_bytes; }
    void Load_from_host(de::Matrix<T>& src) override            /* GPU_Matrix.h:334-343 */
    {
        _MatrixT<T>& s = dynamic_cast<_MatrixT<T>&>(src);
        if (s.width != width || s.height != height) return;
        decxb_memcpy2d(cuP.ctx, Mat.get(), (size_t)pitch * sizeof(T), s.Mat.get(), (size_t)s.pitch * sizeof(T),
                       (size_t)width * sizeof(T), height, 1);
    }
    void Load_to_host(de::Matrix<T>& dst) override              /* GPU_Matrix.h:345-354 */
    {
        _MatrixT<T>& d = dynamic_cast<_MatrixT<T>&>(dst);
        if (d.width != width || d.height != height) return;
        decxb_memcpy2d(cuP.ctx, d.Mat.get(), (size_t)d.pitch * sizeof(T), Mat.get(), (size_t)pitch * sizeof(T),
                       (size_t)width * sizeof(T), height, 2);
    }
    void release() override { Mat.reset(); }
    de::GPU_Matrix<T>& operator=(de::GPU_Matrix<T>& src) override
    {
        _GPU_MatrixT& s = dynamic_cast<_GPU_MatrixT&>(src);
        _attribute_assign(s.width, s.height);
        Mat = s.Mat;
        return *this;
    }
};
using _GPU_Matrix = _GPU_MatrixT<float>;
using _GPU_MatrixH = _GPU_MatrixT<de::Half>;

/* ---- Tensor / TensorArray (host and device share the geometry) ------------------------------------ */
struct TensorGeom {
    uint width = 0, height = 0, depth = 0, tensor_num = 1, dpitch = 0, wpitch = 0;
    size_t dp_x_wp = 0, _gap = 0, element_num = 0, _element_num = 0, total_bytes = 0;
    void assign(uint w, uint h, uint d, uint n)
    {
        width = w; height = h; depth = d; tensor_num = n;
        wpitch = ceil_to(w, 4); dpitch = ceil_to(d, 4);             /* Tensor.h:162-184, TensorArray.h:174-198 */
        dp_x_wp = (size_t)dpitch * wpitch;
        _gap = dp_x_wp * h;
        element_num = (size_t)d * w * h * n;
        _element_num = _gap * n;
        total_bytes = _element_num * sizeof(float);
    }
};

class _Tensor : public de::Tensor<float>, public TensorGeom {
public:
    int _store_type = Page_Default;
    std::shared_ptr<float> Tens;
    void construct(uint w, uint h, uint d, int store) { assign(w, h, d, 1); _store_type = store; Tens = host_block(total_bytes, store); }
    void re_construct(uint w, uint h, uint d, int store)
    {
        if (w != width || h != height || d != depth || store != _store_type || !Tens) construct(w, h, d, store);
    }
    _Tensor() { assign(0, 0, 0, 1); }
    _Tensor(uint w, uint h, uint d, int store) { construct(w, h, d, store); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    uint Depth() override { return depth; }
    float& index(const int x, const int y, const int z) override
    {
        return Tens.get()[(size_t)x * dp_x_wp + (size_t)y * dpitch + (size_t)z];   /* x = row, y = column */
    }
    de::Tensor<float>& operator=(de::Tensor<float>& src) override
    {
        _Tensor& s = dynamic_cast<_Tensor&>(src);
        assign(s.width, s.height, s.depth, 1); _store_type = s._store_type; Tens = s.Tens;
        return *this;
    }
    void release() override { Tens.reset(); }
};

class _TensorArray : public de::TensorArray<float>, public TensorGeom {
public:
    int _store_type = Page_Default;
    std::shared_ptr<float> TensArr;
    void construct(uint w, uint h, uint d, uint n, int store) { assign(w, h, d, n); _store_type = store; TensArr = host_block(total_bytes, store); }
    void re_construct(uint w, uint h, uint d, uint n, int store)
    {
        if (w != width || h != height || d != depth || n != tensor_num || store != _store_type || !TensArr) construct(w, h, d, n, store);
    }
    _TensorArray() { assign(0, 0, 0, 0); }
    _TensorArray(uint w, uint h, uint d, uint n, int store) { construct(w, h, d, n, store); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    uint Depth() override { return depth; }
    uint TensorNum() override { return tensor_num; }
    float& index(const int x, const int y, const int z, const int tensor_id) override
    {
        return TensArr.get()[(size_t)tensor_id * _gap + (size_t)x * dp_x_wp + (size_t)y * dpitch + (size_t)z];
    }
    de::TensorArray<float>& operator=(de::TensorArray<float>& src) override
    {
        _TensorArray& s = dynamic_cast<_TensorArray&>(src);
        assign(s.width, s.height, s.depth, s.tensor_num); _store_type = s._store_type; TensArr = s.TensArr;
        return *this;
    }
    void release() override { TensArr.reset(); }
};

class _GPU_Tensor : public de::GPU_Tensor<float>, public TensorGeom {
public:
    std::shared_ptr<float> Tens;
    void construct(uint w, uint h, uint d) { assign(w, h, d, 1); Tens = device_block(total_bytes); }
    void re_construct(uint w, uint h, uint d) { if (w != width || h != height || d != depth || !Tens) construct(w, h, d); }
    _GPU_Tensor() { assign(0, 0, 0, 1); }
    _GPU_Tensor(uint w, uint h, uint d) { construct(w, h, d); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    uint Depth() override { return depth; }
    de::GPU_Tensor<float>& operator=(de::GPU_Tensor<float>& src) override
    {
        _GPU_Tensor& s = dynamic_cast<_GPU_Tensor&>(src);
        assign(s.width, s.height, s.depth, 1); Tens = s.Tens;
        return *this;
    }
    void Load_from_host(de::Tensor<float>& src) override             /* flat copy, GPU_Tensor.h:355-362 */
    {
        _Tensor& s = dynamic_cast<_Tensor&>(src);
        if (s.total_bytes != total_bytes) return;
        decxb_memcpy2d(cuP.ctx, Tens.get(), total_bytes, s.Tens.get(), total_bytes, total_bytes, 1, 1);
    }
    void Load_to_host(de::Tensor<float>& dst) override
    {
        _Tensor& d = dynamic_cast<_Tensor&>(dst);
        if (d.total_bytes != total_bytes) return;
        decxb_memcpy2d(cuP.ctx, d.Tens.get(), total_bytes, Tens.get(), total_bytes, total_bytes, 1, 2);
    }
    void release() override { Tens.reset(); }
};

class _GPU_TensorArray : public de::GPU_TensorArray<float>, public TensorGeom {
public:
    std::shared_ptr<float> TensArr;
    void construct(uint w, uint h, uint d, uint n) { assign(w, h, d, n); TensArr = device_block(total_bytes); }
    void re_construct(uint w, uint h, uint d, uint n)
    {
        if (w != width || h != height || d != depth || n != tensor_num || !TensArr) construct(w, h, d, n);
    }
    _GPU_TensorArray() { assign(0, 0, 0, 0); }
    _GPU_TensorArray(uint w, uint h, uint d, uint n) { construct(w, h, d, n); }
    uint Width() override { return width; }
    uint Height() override { return height; }
    uint Depth() override { return depth; }
    uint TensorNum() override { return tensor_num; }
    void Load_from_host(de::TensorArray<float>& src) override
    {
        _TensorArray& s = dynamic_cast<_TensorArray&>(src);
        if (s.total_bytes != total_bytes) return;
        decxb_memcpy2d(cuP.ctx, TensArr.get(), total_bytes, s.TensArr.get(), total_bytes, total_bytes, 1, 1);
    }
    void Load_to_host(de::TensorArray<float>& dst) override
    {
        _TensorArray& d = dynamic_cast<_TensorArray&>(dst);
        if (d.total_bytes != total_bytes) return;
        decxb_memcpy2d(cuP.ctx, d.TensArr.get(), total_bytes, TensArr.get(), total_bytes, total_bytes, 1, 2);
    }
    de::GPU_TensorArray<float>& operator=(de::GPU_TensorArray<float>& src) override
    {
        _GPU_TensorArray& s = dynamic_cast<_GPU_TensorArray&>(src);
        assign(s.width, s.height, s.depth, s.tensor_num); TensArr = s.TensArr;
        return *this;
    }
    void release() override { TensArr.reset(); }
};

}  // namespace decx

/* ---- factories: objects are new-ed and owned by the caller, as in the reference
 *      (srcs/classes/Matrix.h:421-476; the user calls release()) ------------------------------------ */
namespace de {
template <> Matrix<float>& CreateMatrixRef<float>() { return *(new decx::_Matrix()); }
template <> Matrix<float>* CreateMatrixPtr<float>() { return new decx::_Matrix(); }
template <> Matrix<float>& CreateMatrixRef<float>(const uint w, const uint h, const int st) { return *(new decx::_Matrix(w, h, st)); }
template <> Matrix<float>* CreateMatrixPtr<float>(const uint w, const uint h, const int st) { return new decx::_Matrix(w, h, st); }
template <> MatrixArray<float>& CreateMatrixArrayRef<float>() { return *(new decx::_MatrixArray()); }
template <> MatrixArray<float>* CreateMatrixArrayPtr<float>() { return new decx::_MatrixArray(); }
template <> MatrixArray<float>& CreateMatrixArrayRef<float>(uint w, uint h, uint n, const int f) { return *(new decx::_MatrixArray(w, h, n, f)); }
template <> MatrixArray<float>* CreateMatrixArrayPtr<float>(uint w, uint h, uint n, const int f) { return new decx::_MatrixArray(w, h, n, f); }
template <> Matrix<Half>& CreateMatrixRef<Half>() { return *(new decx::_MatrixH()); }
template <> Matrix<Half>* CreateMatrixPtr<Half>() { return new decx::_MatrixH(); }
template <> Matrix<Half>& CreateMatrixRef<Half>(const uint w, const uint h, const int st) { return *(new decx::_MatrixH(w, h, st)); }
template <> Matrix<Half>* CreateMatrixPtr<Half>(const uint w, const uint h, const int st) { return new decx::_MatrixH(w, h, st); }
template <> GPU_Matrix<Half>& CreateGPUMatrixRef<Half>() { return *(new decx::_GPU_MatrixH()); }
template <> GPU_Matrix<Half>* CreateGPUMatrixPtr<Half>() { return new decx::_GPU_MatrixH(); }
template <> GPU_Matrix<Half>& CreateGPUMatrixRef<Half>(const uint w, const uint h) { return *(new decx::_GPU_MatrixH(w, h)); }
template <> GPU_Matrix<Half>* CreateGPUMatrixPtr<Half>(const uint w, const uint h) { return new decx::_GPU_MatrixH(w, h); }
template <> GPU_Matrix<float>& CreateGPUMatrixRef<float>() { return *(new decx::_GPU_Matrix()); }
template <> GPU_Matrix<float>* CreateGPUMatrixPtr<float>() { return new decx::_GPU_Matrix(); }
template <> GPU_Matrix<float>& CreateGPUMatrixRef<float>(const uint w, const uint h) { return *(new decx::_GPU_Matrix(w, h)); }
template <> GPU_Matrix<float>* CreateGPUMatrixPtr<float>(const uint w, const uint h) { return new decx::_GPU_Matrix(w, h); }
template <> Tensor<float>& CreateTensorRef<float>() { return *(new decx::_Tensor()); }
template <> Tensor<float>* CreateTensorPtr<float>() { return new decx::_Tensor(); }
template <> Tensor<float>& CreateTensorRef<float>(const uint w, const uint h, const uint d, const int f) { return *(new decx::_Tensor(w, h, d, f)); }
template <> Tensor<float>* CreateTensorPtr<float>(const uint w, const uint h, const uint d, const int f) { return new decx::_Tensor(w, h, d, f); }
template <> GPU_Tensor<float>& CreateGPUTensorRef<float>() { return *(new decx::_GPU_Tensor()); }
template <> GPU_Tensor<float>* CreateGPUTensorPtr<float>() { return new decx::_GPU_Tensor(); }
template <> GPU_Tensor<float>& CreateGPUTensorRef<float>(const uint w, const uint h, const uint d) { return *(new decx::_GPU_Tensor(w, h, d)); }
template <> GPU_Tensor<float>* CreateGPUTensorPtr<float>(const uint w, const uint h, const uint d) { return new decx::_GPU_Tensor(w, h, d); }
template <> TensorArray<float>& CreateTensorArrayRef<float>() { return *(new decx::_TensorArray()); }
template <> TensorArray<float>* CreateTensorArrayPtr<float>() { return new decx::_TensorArray(); }
template <> TensorArray<float>& CreateTensorArrayRef<float>(const uint w, const uint h, const uint d, const uint n, const int st) { return *(new decx::_TensorArray(w, h, d, n, st)); }
template <> TensorArray<float>* CreateTensorArrayPtr<float>(const uint w, const uint h, const uint d, const uint n, const int st) { return new decx::_TensorArray(w, h, d, n, st); }
template <> GPU_TensorArray<float>& CreateGPUTensorArrayRef<float>() { return *(new decx::_GPU_TensorArray()); }
template <> GPU_TensorArray<float>* CreateGPUTensorArrayPtr<float>() { return new decx::_GPU_TensorArray(); }
template <> GPU_TensorArray<float>& CreateGPUTensorArrayRef<float>(const uint w, const uint h, const uint d, const uint n) { return *(new decx::_GPU_TensorArray(w, h, d, n)); }
template <> GPU_TensorArray<float>* CreateGPUTensorArrayPtr<float>(const uint w, const uint h, const uint d, const uint n) { return new decx::_GPU_TensorArray(w, h, d, n); }

void InitCuda()
{
    if (decx::cuP.is_init) return;
    if (decxb_init(0, &decx::cuP.ctx) == DECXB_OK) decx::cuP.is_init = true;
}

void release_all_tmp()
{
    if (decx::cuP.ctx) decxb_release_cached(decx::cuP.ctx);
}

namespace cuda {

void SetGemmPlainTF32(bool on) { decx::cuP.plain_tf32 = on; }
void SetGemmStrictAccumulation(bool on) { decx::cuP.strict = on; }
void SetConvExplicitPack(bool on) { decx::cuP.explicit_pack = on; }

static int gemm_mode()
{
    return decx::cuP.plain_tf32 ? DECXB_GEMM_1XTF32 : decx::cuP.strict ? DECXB_GEMM_3XTF32_STRICT : DECXB_GEMM_3XTF32;
}
static int conv_gemm_mode() { return gemm_mode(); }
static int conv_algo() { return decx::cuP.explicit_pack ? DECXB_CONV_EXPLICIT : DECXB_CONV_IMPLICIT; }

static DH gemm_host(Matrix<float>& A, Matrix<float>& B, Matrix<float>* C, Matrix<float>& dst)
{
    DH handle;
    decx::_Matrix& _A = dynamic_cast<decx::_Matrix&>(A);
    decx::_Matrix& _B = dynamic_cast<decx::_Matrix&>(B);
    decx::_Matrix* _C = C ? dynamic_cast<decx::_Matrix*>(C) : nullptr;
    decx::_Matrix& _dst = dynamic_cast<decx::_Matrix&>(dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_A.width != _B.height) { decx::MDim_Not_Matching(&handle); return handle; }
    if (_C && (_C->width != _B.width || _C->height != _A.height)) { decx::MDim_Not_Matching(&handle); return handle; }
    _dst.re_construct(_B.width, _A.height, decx::Page_Locked);
    int rc = decxb_gemm_f32_host(decx::cuP.ctx, gemm_mode(), DECXB_TILE_AUTO, _A.height, _B.width, _A.width,
                                 _A.Mat.get(), _A.pitch, _B.Mat.get(), _B.pitch,
                                 _C ? _C->Mat.get() : nullptr, _C ? _C->pitch : 0, _dst.Mat.get(), _dst.pitch);
    decx::from_status(&handle, rc);
    return handle;
}

static DH gemm_dev(GPU_Matrix<float>& A, GPU_Matrix<float>& B, GPU_Matrix<float>* C, GPU_Matrix<float>& dst)
{
    DH handle;
    decx::_GPU_Matrix& _A = dynamic_cast<decx::_GPU_Matrix&>(A);
    decx::_GPU_Matrix& _B = dynamic_cast<decx::_GPU_Matrix&>(B);
    decx::_GPU_Matrix* _C = C ? dynamic_cast<decx::_GPU_Matrix*>(C) : nullptr;
    decx::_GPU_Matrix& _dst = dynamic_cast<decx::_GPU_Matrix&>(dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_A.width != _B.height) { decx::MDim_Not_Matching(&handle); return handle; }
    if (_C && (_C->width != _B.width || _C->height != _A.height)) { decx::MDim_Not_Matching(&handle); return handle; }
    _dst.re_construct(_B.width, _A.height);
    int rc = decxb_gemm_f32(decx::cuP.ctx, gemm_mode(), DECXB_TILE_AUTO, _A.height, _B.width, _A.width,
                            _A.Mat.get(), _A.pitch, _B.Mat.get(), _B.pitch,
                            _C ? _C->Mat.get() : nullptr, _C ? _C->pitch : 0, _dst.Mat.get(), _dst.pitch, nullptr);
    if (rc == DECXB_OK) rc = decxb_synchronize(decx::cuP.ctx);       /* blocking, like the reference (GEMM.h:449) */
    decx::from_status(&handle, rc);
    return handle;
}

DH GEMM(Matrix<float>& A, Matrix<float>& B, Matrix<float>& dst) { return gemm_host(A, B, nullptr, dst); }
DH GEMM(Matrix<float>& A, Matrix<float>& B, Matrix<float>& C, Matrix<float>& dst) { return gemm_host(A, B, &C, dst); }
DH GEMM(GPU_Matrix<float>& A, GPU_Matrix<float>& B, GPU_Matrix<float>& dst) { return gemm_dev(A, B, nullptr, dst); }
DH GEMM(GPU_Matrix<float>& A, GPU_Matrix<float>& B, GPU_Matrix<float>& C, GPU_Matrix<float>& dst) { return gemm_dev(A, B, &C, dst); }

static DH gemm_host_h(Matrix<Half>& A, Matrix<Half>& B, Matrix<Half>* C, Matrix<Half>& dst)
{
    DH handle;
    decx::_MatrixH& _A = dynamic_cast<decx::_MatrixH&>(A);
    decx::_MatrixH& _B = dynamic_cast<decx::_MatrixH&>(B);
    decx::_MatrixH* _C = C ? dynamic_cast<decx::_MatrixH*>(C) : nullptr;
    decx::_MatrixH& _dst = dynamic_cast<decx::_MatrixH&>(dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_A.width != _B.height) { decx::MDim_Not_Matching(&handle); return handle; }
    if (_C && (_C->width != _B.width || _C->height != _A.height)) { decx::MDim_Not_Matching(&handle); return handle; }
    _dst.re_construct(_B.width, _A.height, decx::Page_Locked);
    int rc = decxb_gemm_f16_host(decx::cuP.ctx, _A.height, _B.width, _A.width, _A.Mat.get(), _A.pitch, _B.Mat.get(), _B.pitch,
                                 _C ? _C->Mat.get() : nullptr, _C ? _C->pitch : 0, _dst.Mat.get(), _dst.pitch);
    decx::from_status(&handle, rc);
    return handle;
}

static DH gemm_dev_h(GPU_Matrix<Half>& A, GPU_Matrix<Half>& B, GPU_Matrix<Half>* C, GPU_Matrix<Half>& dst)
{
    DH handle;
    decx::_GPU_MatrixH& _A = dynamic_cast<decx::_GPU_MatrixH&>(A);
    decx::_GPU_MatrixH& _B = dynamic_cast<decx::_GPU_MatrixH&>(B);
    decx::_GPU_MatrixH* _C = C ? dynamic_cast<decx::_GPU_MatrixH*>(C) : nullptr;
    decx::_GPU_MatrixH& _dst = dynamic_cast<decx::_GPU_MatrixH&>(dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_A.width != _B.height) { decx::MDim_Not_Matching(&handle); return handle; }
    if (_C && (_C->width != _B.width || _C->height != _A.height)) { decx::MDim_Not_Matching(&handle); return handle; }
    _dst.re_construct(_B.width, _A.height);
    int rc = decxb_gemm_f16(decx::cuP.ctx, _A.height, _B.width, _A.width, _A.Mat.get(), _A.pitch, _B.Mat.get(), _B.pitch,
                            _C ? _C->Mat.get() : nullptr, _C ? _C->pitch : 0, _dst.Mat.get(), _dst.pitch, nullptr);
    if (rc == DECXB_OK) rc = decxb_synchronize(decx::cuP.ctx);
    decx::from_status(&handle, rc);
    return handle;
}

DH GEMM(Matrix<Half>& A, Matrix<Half>& B, Matrix<Half>& dst) { return gemm_host_h(A, B, nullptr, dst); }
DH GEMM(Matrix<Half>& A, Matrix<Half>& B, Matrix<Half>& C, Matrix<Half>& dst) { return gemm_host_h(A, B, &C, dst); }
DH GEMM(GPU_Matrix<Half>& A, GPU_Matrix<Half>& B, GPU_Matrix<Half>& dst) { return gemm_dev_h(A, B, nullptr, dst); }
DH GEMM(GPU_Matrix<Half>& A, GPU_Matrix<Half>& B, GPU_Matrix<Half>& C, GPU_Matrix<Half>& dst) { return gemm_dev_h(A, B, &C, dst); }

static DH gemm3(MatrixArray<float>& A, MatrixArray<float>& B, MatrixArray<float>* C, MatrixArray<float>& dst)
{
    DH handle;
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    decx::_MatrixArray* _A = dynamic_cast<decx::_MatrixArray*>(&A);
    decx::_MatrixArray* _B = dynamic_cast<decx::_MatrixArray*>(&B);
    decx::_MatrixArray* _C = C ? dynamic_cast<decx::_MatrixArray*>(C) : nullptr;
    decx::_MatrixArray* _dst = dynamic_cast<decx::_MatrixArray*>(&dst);
    if (_A->ArrayNumber != _B->ArrayNumber || (_C && _C->ArrayNumber != _A->ArrayNumber)) {
        decx::set_handle(&handle, decx::DECX_FAIL_MNumNotMatching, "The number of matrices don't match each other");
        return handle;
    }
    if (_A->width != _B->height || (_C && (_C->width != _B->width || _C->height != _A->height))) {
        decx::MDim_Not_Matching(&handle); return handle;
    }
    _dst->re_construct(_B->width, _A->height, (uint)_A->ArrayNumber, decx::Page_Locked);
    int rc = decxb_gemm_f32_batched_host(decx::cuP.ctx, conv_gemm_mode(), DECXB_TILE_AUTO, (int64_t)_A->ArrayNumber,
                                         _A->height, _B->width, _A->width,
                                         _A->MatArr.get(), _A->pitch, (int64_t)_A->_plane,
                                         _B->MatArr.get(), _B->pitch, (int64_t)_B->_plane,
                                         _C ? _C->MatArr.get() : nullptr, _C ? _C->pitch : 0, _C ? (int64_t)_C->_plane : 0,
                                         _dst->MatArr.get(), _dst->pitch, (int64_t)_dst->_plane);
    decx::from_status(&handle, rc);
    return handle;
}

DH GEMM3(MatrixArray<float>& A, MatrixArray<float>& B, MatrixArray<float>& dst) { return gemm3(A, B, nullptr, dst); }
DH GEMM3(MatrixArray<float>& A, MatrixArray<float>& B, MatrixArray<float>& C, MatrixArray<float>& dst) { return gemm3(A, B, &C, dst); }

DH Conv2_MK_im2col(Tensor<float>& src, TensorArray<float>& kernel, Tensor<float>& dst, const int flag)
{
    DH handle;
    decx::_Tensor* _src = dynamic_cast<decx::_Tensor*>(&src);
    decx::_TensorArray* _kernel = dynamic_cast<decx::_TensorArray*>(&kernel);
    decx::_Tensor* _dst = dynamic_cast<decx::_Tensor*>(&dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_src->depth != _kernel->depth) { decx::TDim_Not_Matching(&handle); return handle; }
    decxb_conv_geom g;
    int rc = decxb_conv_geometry(_src->width, _src->height, _src->depth, _kernel->width, _kernel->height, _kernel->tensor_num, flag, &g);
    if (rc) { decx::from_status(&handle, rc); return handle; }
    _dst->re_construct((uint)g.out_w, (uint)g.out_h, _kernel->tensor_num, decx::Page_Locked);   /* conv2_mk_im2col.h:173-178 */
    rc = decxb_conv2_im2col_f32_host(decx::cuP.ctx, conv_gemm_mode(), conv_algo(), flag,
                                     _src->Tens.get(), _src->width, _src->height, _src->depth,
                                     _kernel->TensArr.get(), _kernel->width, _kernel->height, _kernel->tensor_num,
                                     _dst->Tens.get(), 1, 0, 0);
    decx::from_status(&handle, rc);
    return handle;
}

static DH conv_dev(const float* src, uint W, uint H, uint depth, int64_t batch, decx::_GPU_TensorArray* k, float* dst, int flag)
{
    DH handle;
    int rc = decxb_conv2_im2col_f32(decx::cuP.ctx, conv_gemm_mode(), conv_algo(), flag, src, W, H, depth,
                                    k->TensArr.get(), k->width, k->height, k->tensor_num, dst, batch, 0, 0, nullptr);
    if (rc == DECXB_OK) rc = decxb_synchronize(decx::cuP.ctx);
    decx::from_status(&handle, rc);
    return handle;
}

DH Conv2_MK_im2col(GPU_Tensor<float>& src, GPU_TensorArray<float>& kernel, GPU_Tensor<float>& dst, const int flag)
{
    DH handle;
    decx::_GPU_Tensor* _src = dynamic_cast<decx::_GPU_Tensor*>(&src);
    decx::_GPU_TensorArray* _kernel = dynamic_cast<decx::_GPU_TensorArray*>(&kernel);
    decx::_GPU_Tensor* _dst = dynamic_cast<decx::_GPU_Tensor*>(&dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_src->depth != _kernel->depth) { decx::TDim_Not_Matching(&handle); return handle; }
    decxb_conv_geom g;
    int rc = decxb_conv_geometry(_src->width, _src->height, _src->depth, _kernel->width, _kernel->height, _kernel->tensor_num, flag, &g);
    if (rc) { decx::from_status(&handle, rc); return handle; }
    _dst->re_construct((uint)g.out_w, (uint)g.out_h, _kernel->tensor_num);
    return conv_dev(_src->Tens.get(), _src->width, _src->height, _src->depth, 1, _kernel, _dst->Tens.get(), flag);
}

DH Conv2_MK_im2col(GPU_TensorArray<float>& src, GPU_TensorArray<float>& kernel, GPU_TensorArray<float>& dst, const int flag)
{
    DH handle;
    decx::_GPU_TensorArray* _src = dynamic_cast<decx::_GPU_TensorArray*>(&src);
    decx::_GPU_TensorArray* _kernel = dynamic_cast<decx::_GPU_TensorArray*>(&kernel);
    decx::_GPU_TensorArray* _dst = dynamic_cast<decx::_GPU_TensorArray*>(&dst);
    if (!decx::cuP.is_init) { decx::Not_init(&handle); return handle; }
    if (_src->depth != _kernel->depth) { decx::TDim_Not_Matching(&handle); return handle; }
    decxb_conv_geom g;
    int rc = decxb_conv_geometry(_src->width, _src->height, _src->depth, _kernel->width, _kernel->height, _kernel->tensor_num, flag, &g);
    if (rc) { decx::from_status(&handle, rc); return handle; }
    _dst->re_construct((uint)g.out_w, (uint)g.out_h, _kernel->tensor_num, _src->tensor_num);
    return conv_dev(_src->TensArr.get(), _src->width, _src->height, _src->depth, _src->tensor_num, _kernel, _dst->TensArr.get(), flag);
}

}  // namespace cuda
}  // namespace de
