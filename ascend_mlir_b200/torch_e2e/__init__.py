"""Torch module -> verified GPU kernel, as a pytest decorator (the reference's python/torch/framework package).

    from ascend_mlir_b200.torch_e2e import torch_e2e_test, TensorSpec

    @torch_e2e_test
    def test_my_model():
        class Model(torch.nn.Module):
            def forward(self, x, y):
                return (x + y).sum(dim=1)
        return Model(), [TensorSpec(("M", "N"), torch.float16)] * 2
"""
from .pipeline import PipelineError, compile_model, run_autotuner, torch_e2e_test
from .tensor_spec import TensorSpec
from .torch2linalg import UnsupportedTorchOp, torch_to_linalg, torch_to_linalg_with_state

__all__ = ["torch_e2e_test", "TensorSpec", "torch_to_linalg", "torch_to_linalg_with_state", "compile_model", "run_autotuner", "PipelineError",
           "UnsupportedTorchOp"]
