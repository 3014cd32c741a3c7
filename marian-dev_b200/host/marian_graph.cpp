// See marian_graph.h.  Everything numeric happens in libmarian_i8.so; this file is graph plumbing.
#include "marian_graph.h"

#include <cuda_runtime.h>

#include "../../include/marian_i8.h"
#include "../../include/marian_packed8.h"

namespace marian {

namespace {
void check(int rc, const char* what) {
  if(rc != MI8_OK)
    MI8_ABORT(std::string("int8 engine, ") + what + ": " + mi8_strerror(rc));
}
void checkCuda(cudaError_t e, const char* what) {
  if(e != cudaSuccess)
    MI8_ABORT(std::string("CUDA, ") + what + ": " + cudaGetErrorString(e));
}
cudaStream_t streamOf(const ExpressionGraph* g) { return g->stream() ? static_cast<cudaStream_t>(g->stream()) : cudaStreamPerThread; }
}  // namespace

std::string typeName(Type t) {
  switch(t) {
    case Type::int8: return "int8";
    case Type::float32: return "float32";
    case Type::intgemm8: return "intgemm8";
    case Type::intgemm16: return "intgemm16";
    case Type::packed8avx2: return "packed8avx2";
    case Type::packed8avx512: return "packed8avx512";
  }
  return "unknown";
}

namespace {
size_t packed8ItemBytes(const Shape& shape) { return (mi8p_packed_bytes(shape[-2], shape[-1]) + 255) / 256 * 256; }
}  // namespace

size_t requiredBytes(const Shape& shape, Type type) {
  if(isPacked(type))
    return packed8ItemBytes(shape) + shape.elements();
  if(isIntgemm(type))
    return shape.elements() * sizeOf(type) + sizeOf(Type::float32);
  return shape.elements() * sizeOf(type);
}

ExpressionGraph::ExpressionGraph(void* arena, size_t arenaBytes, void* workspace, size_t workspaceBytes, void* stream)
    : arena_(static_cast<uint8_t*>(arena)), arenaBytes_(arenaBytes), ws_(workspace), wsBytes_(workspaceBytes), stream_(stream) {
  MI8_ABORT_IF(arena == nullptr || (reinterpret_cast<uintptr_t>(arena) & 255u), "Graph arena must be a 256-byte aligned device pointer");
  MI8_ABORT_IF(workspace == nullptr || workspaceBytes < mi8_workspace_bytes(0, 0, 0), "Graph workspace too small");
  check(mi8_workspace_init(ws_, wsBytes_, stream_), "workspace init");
}

Tensor ExpressionGraph::allocate(const Shape& shape, Type type) {
  const size_t bytes = (requiredBytes(shape, type) + 255) / 256 * 256;
  MI8_ABORT_IF(used_ + bytes > arenaBytes_, "Out of graph memory");
  Tensor t = std::make_shared<TensorBase>();
  t->memory = arena_ + used_;
  t->shape = shape;
  t->type = type;
  used_ += bytes;
  return t;
}

Expr ExpressionGraph::param(const std::string& name, const Shape& shape, Type type, const void* hostData) {
  Expr n = std::make_shared<Node>();
  n->graph = this;
  n->name = name;
  n->shapeValue = shape;
  n->typeValue = type;
  n->value = allocate(shape, type);
  checkCuda(cudaMemcpyAsync(n->value->memory, hostData, requiredBytes(shape, type), cudaMemcpyHostToDevice, streamOf(this)), "parameter upload");
  checkCuda(cudaStreamSynchronize(streamOf(this)), "parameter upload");
  return n;
}

Expr ExpressionGraph::constant(const Shape& shape, const std::vector<float>& values) {
  MI8_ABORT_IF(values.size() != shape.elements(), "Constant has the wrong number of values");
  return param("", shape, Type::float32, values.data());
}

Expr ExpressionGraph::intgemm8Param(const std::string& name, Expr w, bool wIsNK) {
  MI8_ABORT_IF(!isFloat(w->value_type()) || w->shape().size() != 2, "Only 2-D float32 parameters can be converted to intgemm8");
  const int k = wIsNK ? w->shape()[1] : w->shape()[0], n = wIsNK ? w->shape()[0] : w->shape()[1];
  Expr q = std::make_shared<Node>();
  q->graph = this;
  q->name = name;
  q->shapeValue = Shape({k, n});  // the logical shape stays [K,N] (expression_graph_packable.h:242-250)
  q->typeValue = Type::intgemm8;
  q->value = allocate(q->shapeValue, Type::intgemm8);
  check(mi8_prepare_b_f32(w->val()->data<float>(), k, n, wIsNK ? 1 : 0, q->value->data<int8_t>(), quantMultPtr(q->value), ws_, wsBytes_,
                          stream_),
        "weight conversion");
  return q;
}

Expr ExpressionGraph::packed8Item(const std::string& name, const Shape& shape, const void* hostItem) {
  MI8_ABORT_IF(shape.size() != 2, "A packed8avx512 parameter is a matrix");
  const int k = shape[0], n = shape[1];
  Expr q = std::make_shared<Node>();
  q->graph = this;
  q->name = name;
  q->shapeValue = shape;
  q->typeValue = Type::packed8avx512;
  q->value = allocate(shape, Type::packed8avx512);
  int8_t* item = q->value->data<int8_t>();
  if(hostItem != nullptr)
    checkCuda(cudaMemcpyAsync(item, hostItem, mi8p_packed_bytes(k, n), cudaMemcpyHostToDevice, streamOf(this)), "parameter upload");
  check(mi8p_unpack_b(item, k, n, item + packed8ItemBytes(shape), stream_), "packed8avx512 load");
  checkCuda(cudaStreamSynchronize(streamOf(this)), "parameter upload");
  return q;
}

Expr ExpressionGraph::packed8Param(const std::string& name, Expr w) {
  MI8_ABORT_IF(!isFloat(w->value_type()) || w->shape().size() != 2, "Only 2-D float32 parameters can be packed");
  const int k = w->shape()[0], n = w->shape()[1];
  Expr q = std::make_shared<Node>();
  q->graph = this;
  q->name = name;
  q->shapeValue = w->shape();
  q->typeValue = Type::packed8avx512;
  q->value = allocate(q->shapeValue, Type::packed8avx512);
  int8_t* item = q->value->data<int8_t>();
  check(mi8p_prepare_b_f32(w->val()->data<float>(), k, n, item, stream_), "packed8avx512 conversion");
  check(mi8p_unpack_b(item, k, n, item + packed8ItemBytes(q->shapeValue), stream_), "packed8avx512 load");
  return q;
}

Expr ExpressionGraph::add(Expr node) {
  node->graph = this;
  tape_.push_back(node);
  return node;
}

void ExpressionGraph::forward() {
  for(; done_ < tape_.size(); ++done_) {
    Expr n = tape_[done_];
    n->value = allocate(n->shape(), n->value_type());
    n->forward(n, n->children);
  }
  checkCuda(cudaStreamSynchronize(streamOf(this)), "forward");
  int status = 0;
  check(mi8_poll_status(&status), "device status");
}

void ExpressionGraph::get(Expr e, std::vector<float>& host) {
  MI8_ABORT_IF(!isFloat(e->value_type()) || !e->val(), "get() needs a computed float32 node");
  host.resize(e->shape().elements());
  checkCuda(cudaMemcpy(host.data(), e->val()->memory, host.size() * sizeof(float), cudaMemcpyDeviceToHost), "download");
}

void ExpressionGraph::get(Expr e, std::vector<int8_t>& host, float* quantMult) {
  MI8_ABORT_IF(!isIntgemm(e->value_type()) || !e->val(), "get() needs a computed intgemm8 node");
  host.resize(e->shape().elements());
  checkCuda(cudaMemcpy(host.data(), e->val()->memory, host.size(), cudaMemcpyDeviceToHost), "download");
  if(quantMult)
    checkCuda(cudaMemcpy(quantMult, quantMultPtr(e->val()), sizeof(float), cudaMemcpyDeviceToHost), "download");
}

Expr lambda(const std::vector<Expr>& children, Shape shape, Type type, LambdaNodeFunctor fn) {
  MI8_ABORT_IF(children.empty(), "Lambda node needs children");
  Expr n = std::make_shared<Node>();
  n->shapeValue = shape;
  n->typeValue = type;
  n->children = children;
  n->forward = fn;
  return children[0]->graph->add(n);
}

// swaps the last two axes (the reference's transpose(a) with the default axes)
Expr transpose(Expr a) {
  MI8_ABORT_IF(!isFloat(a->value_type()), "transpose expects a float32 tensor, not " + typeName(a->value_type()));
  MI8_ABORT_IF(a->shape().size() < 2, "transpose needs at least two axes");
  Shape outShape = a->shape();
  const int r = a->shape()[-2], c = a->shape()[-1];
  outShape.set(-2, c);
  outShape.set(-1, r);
  auto nodeOp = [=](Expr out, const std::vector<Expr>& ch) {
    Tensor in = ch[0]->val();
    const int batch = static_cast<int>(in->shape.elements() / (static_cast<size_t>(r) * c));
    check(mi8_transpose_f32(in->data<float>(), batch, r, c, out->val()->data<float>(), out->graph->stream()), "transpose");
  };
  return lambda({a}, outShape, Type::float32, nodeOp);
}

namespace gpu {
namespace integer {

Expr prepareA(Expr a) {
  auto nodeOp = [](Expr out, const std::vector<Expr>& children) {
    Tensor in = children[0]->val();
    ExpressionGraph* g = out->graph;
    check(mi8_prepare_a_f32(in->data<float>(), rows(in), cols(in), out->val()->data<int8_t>(), quantMultPtr(out->val()), g->workspace(),
                            g->workspaceBytes(), g->stream()),
          "prepareA");
  };
  return lambda({a}, a->shape(), Type::intgemm8, nodeOp);
}

Expr affineOrDot(Expr a, Expr bQuant, Expr bias, bool transA, bool /*transB*/, float scale, bool relu) {
  MI8_ABORT_IF(!isFloat(a->value_type()), "Intgemm expects type of A to be float32 not " + typeName(a->value_type()));
  MI8_ABORT_IF(!isIntgemm(bQuant->value_type()),
               "Intgemm expects type of B to be a variant of intgemm not " + typeName(bQuant->value_type()));
  MI8_ABORT_IF(bQuant->value_type() != Type::intgemm8, "Only intgemm8 is supported on the GPU, not " + typeName(bQuant->value_type()));
  if(transA)   // as the reference: A is transposed by a node of its own in front of the quantisation (intgemm_interface.h:52)
    a = transpose(a);
  MI8_ABORT_IF(a->shape()[-1] != bQuant->shape()[-2], "Inner dimensions of A and B do not match");
  Expr aQuant = prepareA(a);
  Shape outShape = aQuant->shape();
  outShape.set(-1, bQuant->shape()[-1]);
  auto nodeOp = [=](Expr out, const std::vector<Expr>& ch) {
    Tensor A = ch[0]->val(), B = ch[1]->val();
    const float* b = ch.size() > 2 ? ch[2]->val()->data<float>() : nullptr;
    ExpressionGraph* g = out->graph;
    check(mi8_multiply_i8(A->data<int8_t>(), B->data<int8_t>(), rows(A), B->shape[-1], cols(A), quantMultPtr(A), quantMultPtr(B), scale, b,
                          relu ? 1 : 0, out->val()->data<float>(), MI8_F32, nullptr, g->workspace(), g->workspaceBytes(), g->stream()),
          "multiply");
  };
  std::vector<Expr> children = {aQuant, bQuant};
  if(bias) {
    MI8_ABORT_IF(!isFloat(bias->value_type()) || static_cast<int>(bias->shape().elements()) != bQuant->shape()[-1],
                 "Bias must be float32 with one value per output column");
    children.push_back(bias);
  }
  return lambda(children, outShape, Type::float32, nodeOp);
}

}  // namespace integer

namespace variant {

Expr affine(Type packType, Expr a, Expr bPacked, const Shape& bShape, Expr bias, bool transA, bool transB, float scale) {
  MI8_ABORT_IF(packType != Type::packed8avx512, "Only avx512 packed matrix format is supported, not " + typeName(packType));
  MI8_ABORT_IF(transA || transB, "Transposition is currently not supported");
  MI8_ABORT_IF(scale != 1.f, "The packed int8 product has no scalar factor");
  MI8_ABORT_IF(!isFloat(a->value_type()), "Packed GEMM expects type of A to be float32 not " + typeName(a->value_type()));
  MI8_ABORT_IF(a->shape()[-1] != bShape[-2], "Inner dimensions of A and B do not match");
  Shape outShape = a->shape();
  outShape.set(-1, bShape[-1]);
  const int k = bShape[-2], n = bShape[-1];
  auto nodeOp = [=](Expr out, const std::vector<Expr>& ch) {
    Tensor A = ch[0]->val(), B = ch[1]->val();
    const float* b = ch.size() > 2 ? ch[2]->val()->data<float>() : nullptr;
    ExpressionGraph* g = out->graph;
    const int m = rows(A);
    const int8_t* item = B->data<int8_t>();
    const int8_t* tail = item + static_cast<size_t>(k) * n;   // scaleB, zeroPointB, colOffsetsB (mjdgemm_avx512.cpp:222-227)
    const int8_t* bt = item + packed8ItemBytes(B->shape);
    Shape scratchShape({static_cast<int>(mi8p_scratch_bytes(m, k))});
    Tensor scratch = g->allocate(scratchShape, Type::int8);
    check(mi8p_gemm_int8_packed(A->data<float>(), bt, reinterpret_cast<const float*>(tail), reinterpret_cast<const int32_t*>(tail + 4 * n),
                                reinterpret_cast<const int32_t*>(tail + 8 * n), b, out->val()->data<float>(), m, n, k, scratch->memory,
                                scratchShape.elements(), g->workspace(), g->workspaceBytes(), g->stream()),
          "packed multiply");
  };
  std::vector<Expr> children = {a, bPacked};
  if(bias) {
    MI8_ABORT_IF(!isFloat(bias->value_type()) || static_cast<int>(bias->shape().elements()) != n,
                 "Bias must be float32 with one value per output column");
    children.push_back(bias);
  }
  return lambda(children, outShape, Type::float32, nodeOp);
}

Expr dot(Type packType, Expr a, Expr bPacked, const Shape& bShape, bool transA, bool transB, float scale) {
  return affine(packType, a, bPacked, bShape, nullptr, transA, transB, scale);
}

}  // namespace variant
}  // namespace gpu

Expr dot(Expr a, Expr b, bool transA, bool transB, float scale) {
  if(isFloat(a->value_type()) && isIntgemm(b->value_type()))
    return gpu::integer::affineOrDot(a, b, nullptr, transA, transB, scale);
  if(isFloat(a->value_type()) && isPacked(b->value_type()))
    return gpu::variant::dot(b->value_type(), a, b, b->shape(), transA, transB, scale);
  MI8_ABORT("GPU only supports float for A and intgemm8 for B on this path; float x float products belong to Marian's cuBLAS path");
}

Expr affine(Expr a, Expr b, Expr bias, bool transA, bool transB, float scale) {
  if(isFloat(a->value_type()) && isIntgemm(b->value_type()))
    return gpu::integer::affineOrDot(a, b, bias, transA, transB, scale);
  if(isFloat(a->value_type()) && isPacked(b->value_type()))   // expression_operators.cpp:697-700
    return gpu::variant::affine(b->value_type(), a, b, b->shape(), bias, transA, transB, scale);
  MI8_ABORT("GPU only supports float for A and intgemm8 for B on this path; float x float products belong to Marian's cuBLAS path");
}

Expr affineWithReluDropout(Expr x, Expr W, Expr bias, float dropProb) {
  MI8_ABORT_IF(dropProb != 0.f, "Dropout is a training feature; the int8 path is inference-only");
  if(isFloat(x->value_type()) && isIntgemm(W->value_type()))
    return gpu::integer::affineOrDot(x, W, bias, false, false, 1.f, /*relu=*/true);  // ReLU fused into the write-back
  MI8_ABORT("GPU only supports float for A and intgemm8 for B on this path; float x float products belong to Marian's cuBLAS path");
}

}  // namespace marian
