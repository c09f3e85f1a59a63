// tim::vx::Graph — tensor/operation registry with Compile and Run.
// Restates include/tim/vx/graph.h:49-116 of the reference.  Compile validates
// the graph, infers TRANSIENT shapes and builds the CUDA launch plan; Run
// replays it and returns when the GPU is done.
#ifndef TIM_VX_GRAPH_H_
#define TIM_VX_GRAPH_H_

#include <cstddef>
#include <map>
#include <memory>
#include <vector>

namespace tim {
namespace vx {

class Tensor;
struct TensorSpec;
struct DmaBufferDesc;
class Operation;
class CompileOption;

class Graph {
 public:
  virtual ~Graph() {}

  virtual void SetCompileOption(const CompileOption&) = 0;

  virtual std::shared_ptr<Tensor> CreateTensor(const TensorSpec& spec,
                                               const void* data = nullptr) = 0;
  virtual std::shared_ptr<Tensor> CreateTensor(const TensorSpec& spec,
                                               const DmaBufferDesc& dmafd) = 0;
  // spec.attr_ must be INPUT or OUTPUT; data, when given, is a caller-owned
  // buffer that CopyData*/map() use as the host side of the tensor.
  virtual std::shared_ptr<Tensor> CreateIOTensor(const TensorSpec& spec,
                                                 void* data = nullptr) = 0;
  virtual std::shared_ptr<Tensor> CreateTensorPlaceHolder() = 0;

  virtual bool Compile() = 0;
  // Serialised graphs are a Vivante binary format; not provided (returns false).
  virtual bool CompileToBinary(void* buf, size_t* size) = 0;
  virtual bool Run() = 0;

  template <typename OpType, typename... Params>
  std::shared_ptr<OpType> CreateOperation(Params... parameters) {
    auto op = std::make_shared<OpType>(this, parameters...);
    op_vector_.push_back(op);
    return op;
  }

  virtual const std::vector<std::shared_ptr<Tensor>> InputsTensor() const = 0;
  virtual const std::vector<std::shared_ptr<Tensor>> OutputsTensor() const = 0;

  virtual void UpdateTensorConsumersMap(const std::shared_ptr<Tensor>& tensor,
                                        const Operation* op) = 0;
  virtual void RenewTensorConsumersMap(const std::shared_ptr<Tensor>& org_tensor,
                                       const std::shared_ptr<Tensor>& dst_tensor,
                                       const Operation* op) = 0;
  virtual void UpdateTensorProducerMap(const std::shared_ptr<Tensor>& tensor,
                                       const Operation* op) = 0;
  virtual const std::vector<std::shared_ptr<Operation>> GetConsumersOp(
      std::shared_ptr<Tensor> tensor) const = 0;
  virtual std::shared_ptr<Operation> GetProducerOp(std::shared_ptr<Tensor> tensor) = 0;

  virtual void PrintGraph() const = 0;

  const std::vector<std::shared_ptr<Tensor>> GetConstantInputs() const;
  virtual std::vector<std::shared_ptr<Operation>>& OpVector() = 0;
  virtual std::map<std::shared_ptr<Tensor>, std::vector<std::shared_ptr<Operation>>>&
  TensorConsumer() = 0;
  virtual std::map<std::shared_ptr<Tensor>, std::shared_ptr<Operation>>&
  TensorProducer() = 0;

 protected:
  std::vector<std::shared_ptr<tim::vx::Operation>> op_vector_;
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_GRAPH_H_
