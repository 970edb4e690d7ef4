"""Quantisation-aware training (fake-quant linears) and quantisation-aware distillation.
reference: mindspeed/core/qat/* (W4A16 / W8A16 / W4A4 fake quant), mindspeed/core/distill/* (teacher manager + KL loss)."""
from .fake_quant import FakeQuantLinear, QATConfig, apply_qat, fake_quantize
from .distill import DistillConfig, TeacherManager, distillation_loss

__all__ = ["FakeQuantLinear", "QATConfig", "apply_qat", "fake_quantize", "DistillConfig", "TeacherManager", "distillation_loss"]
