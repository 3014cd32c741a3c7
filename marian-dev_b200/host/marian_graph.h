// C++ host mirror of the slice of Marian's expression-graph interface that the int8 path uses:
// the operators affine / dot / affineWithReluDropout (src/graph/expression_operators.cpp:554-731), the
// inference-only lambda node they are built from (src/graph/node_operators_binary.h:16-80,
// src/graph/expression_operators.cpp:35-43), intgemm8-typed tensors with the multiplier behind the data
// (src/common/types.cpp:32-37, src/tensors/cpu/integer_common.h:101-111), a 256-byte aligned allocator
// over caller-owned device memory (src/tensors/tensor_allocator.h:17) and a tape that runs forward in
// construction order (src/graph/expression_graph.cpp:130-185).  The node functors unpack tensors into
// raw pointers and call the C ABI of marian_i8.h, exactly what a GPU twin of
// src/tensors/cpu/intgemm_interface.h would do inside Marian.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace marian {

// ABORT with exceptions switched on (setThrowExceptionOnAbort(true), src/common/logging.h:100-140)
class MarianRuntimeException : public std::runtime_error {
public:
  explicit MarianRuntimeException(const std::string& msg) : std::runtime_error(msg) {}
};
#define MI8_ABORT(msg) throw ::marian::MarianRuntimeException(msg)
#define MI8_ABORT_IF(cond, msg) \
  do {                          \
    if(cond)                    \
      MI8_ABORT(msg);           \
  } while(0)

// type tags as stored in binary models (src/common/types.h:270-328)
enum class Type : size_t {
  int8 = 0x0100 + 1,
  float32 = 0x0400 + 4,
  intgemm8 = 0x10000 + 1,
  intgemm16 = 0x10000 + 2,
  packed8avx2 = 0x0800 + 1 + 0x1000,     // FBGEMM int8 items (types.h:313-315); only the avx512 blocking is served
  packed8avx512 = 0x0800 + 1 + 0x2000,
};
inline bool isFloat(Type t) { return (static_cast<size_t>(t) & 0x0400) != 0; }
inline bool isIntgemm(Type t) { return (static_cast<size_t>(t) & 0x10000) != 0; }
inline bool isPacked(Type t) { return (static_cast<size_t>(t) & 0x0800) != 0; }
inline size_t sizeOf(Type t) { return static_cast<size_t>(t) & 0xff; }
std::string typeName(Type t);

struct Shape {
  std::vector<int> dims;
  Shape() {}
  Shape(std::initializer_list<int> d) : dims(d) {}
  size_t size() const { return dims.size(); }
  int operator[](int i) const { return i < 0 ? dims[dims.size() + i] : dims[i]; }
  void set(int i, int v) { (i < 0 ? dims[dims.size() + i] : dims[i]) = v; }
  size_t elements() const {
    size_t n = 1;
    for(int d : dims)
      n *= static_cast<size_t>(d);
    return n;
  }
  bool operator==(const Shape& o) const { return dims == o.dims; }
};

// bytes a tensor needs: intgemm tensors carry one extra float, the quantisation multiplier (types.cpp:32-37);
// a packed8avx512 tensor of logical shape [K,N] holds the item (K*N + 12*N bytes, rounded up to 256) followed by
// the row-major Bt[N,K] copy the GPU multiply reads (made when the parameter is created)
size_t requiredBytes(const Shape& shape, Type type);

struct TensorBase {
  uint8_t* memory = nullptr;  // device pointer
  Shape shape;
  Type type = Type::float32;
  template <typename T>
  T* data() const {
    return reinterpret_cast<T*>(memory);
  }
};
typedef std::shared_ptr<TensorBase> Tensor;

inline int cols(const Tensor& t) { return t->shape[-1]; }
inline int rows(const Tensor& t) { return static_cast<int>(t->shape.elements() / cols(t)); }
// getQuantMult: the float right behind the last quantised element (integer_common.h:101-111)
inline float* quantMultPtr(const Tensor& t) { return reinterpret_cast<float*>(t->memory + t->shape.elements() * sizeOf(t->type)); }

class ExpressionGraph;
struct Node;
typedef std::shared_ptr<Node> Expr;
typedef std::function<void(Expr out, const std::vector<Expr>& children)> LambdaNodeFunctor;

struct Node {
  ExpressionGraph* graph = nullptr;
  Shape shapeValue;
  Type typeValue = Type::float32;
  Tensor value;
  std::vector<Expr> children;
  LambdaNodeFunctor forward;  // empty for parameters and constants
  std::string name;
  const Shape& shape() const { return shapeValue; }
  Type value_type() const { return typeValue; }
  Tensor val() const { return value; }
};

class ExpressionGraph {
public:
  // arena / workspace: caller-owned device memory; stream: cudaStream_t as void* (nullptr = per-thread default)
  ExpressionGraph(void* arena, size_t arenaBytes, void* workspace, size_t workspaceBytes, void* stream = nullptr);

  // parameter with host initial data in the tensor's own layout (for intgemm8: Bt[N,K] then the fp32 multiplier)
  Expr param(const std::string& name, const Shape& shape, Type type, const void* hostData);
  Expr constant(const Shape& shape, const std::vector<float>& values);
  // marian-conv for one parameter: float W[K,N] -> intgemm8 node with logical shape [K,N]
  // (expression_graph_packable.h:160-201); wIsNK: W already is [N,K] (tied embedding used with transB)
  Expr intgemm8Param(const std::string& name, Expr floatParam, bool wIsNK = false);

  // marian-conv --gemm-type packed8avx512 for one parameter (expression_graph_packable.h:49-95): float W[K,N] ->
  // packed8avx512 node, logical shape [K,N]; packed8Item takes the bytes of an item read from a model file instead
  Expr packed8Param(const std::string& name, Expr floatParam);
  Expr packed8Item(const std::string& name, const Shape& shape, const void* hostItem);

  Expr add(Expr node);    // appends a computed node to the tape
  void forward();         // allocate -> forward() per node in tape order, then waits for the stream
  void get(Expr e, std::vector<float>& host);       // copies a float32 value back
  void get(Expr e, std::vector<int8_t>& host, float* quantMult);

  Tensor allocate(const Shape& shape, Type type);   // 256-byte aligned piece of the arena
  void* workspace() const { return ws_; }
  size_t workspaceBytes() const { return wsBytes_; }
  void* stream() const { return stream_; }

private:
  uint8_t* arena_;
  size_t arenaBytes_, used_ = 0;
  void* ws_;
  size_t wsBytes_;
  void* stream_;
  std::vector<Expr> tape_;
  size_t done_ = 0;
};

// inference-only lambda node (expression_operators.cpp:35-43)
Expr lambda(const std::vector<Expr>& children, Shape shape, Type type, LambdaNodeFunctor fn);

// the operator surface of the path (expression_operators.h:489-493,523-528,533-536)
Expr transpose(Expr a);   // last two axes swapped (float32)
Expr dot(Expr a, Expr b, bool transA = false, bool transB = false, float scale = 1.f);
Expr affine(Expr a, Expr b, Expr bias, bool transA = false, bool transB = false, float scale = 1.f);
Expr affineWithReluDropout(Expr x, Expr W, Expr bias, float dropProb = 0.f);

namespace gpu {
namespace integer {
// GPU twins of cpu::integer::prepareA / affineOrDot (src/tensors/cpu/intgemm_interface.h:17-32,46-128)
Expr prepareA(Expr a);
Expr affineOrDot(Expr a, Expr bQuant, Expr bias, bool transA, bool transB, float scale, bool relu = false);
}  // namespace integer
namespace variant {
// GPU twin of cpu::variant::affine / dot for packed int8 weights (src/tensors/cpu/fbgemm/expanded_gemm.h, reached from
// expression_operators.cpp:697-700 when isPacked(b)); the arithmetic is that of mjdgemm::gemmInt8Packed
// (src/tensors/cpu/fbgemm/packed_gemm.cpp:18-31).  `scale` must be 1 and no transposition, as there.
Expr affine(Type packType, Expr a, Expr bPacked, const Shape& bShape, Expr bias, bool transA, bool transB, float scale);
Expr dot(Type packType, Expr a, Expr bPacked, const Shape& bShape, bool transA, bool transB, float scale);
}  // namespace variant
}  // namespace gpu

}  // namespace marian
