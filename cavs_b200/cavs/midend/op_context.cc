#include "cavs/midend/op_context.h"

namespace midend {

int OpContext::dyn_dim_ = -1;

void OpContext::SetTensorOffset() {
  if (!gs_) return;
  const int off = gs_->GetCurrentRoundOffset();
  for (const Tensor* t : inputs_)
    if (t->IsDynamicShape() && !t->IsFullShape()) const_cast<Tensor*>(t)->SetOffsetWithId(off);
  for (Tensor* t : outputs_)
    if (t->IsDynamicShape() && !t->IsFullShape()) t->SetOffsetWithId(off);
}
void OpContext::ResetTensorOffset() {
  for (const Tensor* t : inputs_)
    if (t->IsDynamicShape() && !t->IsFullShape()) const_cast<Tensor*>(t)->SetOffsetWithId(0);
  for (Tensor* t : outputs_)
    if (t->IsDynamicShape() && !t->IsFullShape()) t->SetOffsetWithId(0);
}
void OpContext::ScaleOutputTensor() {
  CHECK(dyn_dim_ > 0) << "SetDynDim was not called";
  for (Tensor* t : outputs_)
    if (t->IsDynamicShape()) t->ScaleDynamicDimension(dyn_dim_);
}
void OpContext::ScaleInputTensor() {
  CHECK(dyn_dim_ > 0) << "SetDynDim was not called";
  for (const Tensor* t : inputs_)
    if (t->IsDynamicShape()) const_cast<Tensor*>(t)->ScaleDynamicDimension(dyn_dim_);
}
void OpContext::SetZero() {
  for (Tensor* t : outputs_)
    if (t->ZeroInitEnforced()) t->InitWithZero(round_);
}
std::string OpContext::debug_info() const {
  std::string s;
  for (const Tensor* t : inputs_) s += "input: " + t->debug_info() + "\n";
  for (Tensor* t : outputs_) s += "output: " + t->debug_info() + "\n";
  return s;
}

}  // namespace midend
