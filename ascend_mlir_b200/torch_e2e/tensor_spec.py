"""Shape pattern of one model input: which dimensions are fixed and which are dynamic.

Same contract as the reference's python/torch/framework/tensor_spec.py:10-59: a dimension is an int (static in
the IR), a str (named dynamic dimension; equal names in different specs are the same symbol) or None (an
anonymous dynamic dimension).  Dynamic dimensions without a requested size are sampled at 64; the default
element type is float16.
"""
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

import torch
from torch.export import Dim

DEFAULT_DYNAMIC_SIZE = 64


@dataclass
class TensorSpec:
    shape: Tuple[Union[int, str, None], ...]
    dtype: torch.dtype = torch.float16

    def concrete_shape(self, dim_sizes: Optional[Dict[str, int]] = None) -> Tuple[int, ...]:
        sizes = dim_sizes or {}
        out = []
        for d in self.shape:
            if isinstance(d, int):
                out.append(d)
            elif isinstance(d, str):
                out.append(int(sizes.get(d, DEFAULT_DYNAMIC_SIZE)))
            else:
                out.append(DEFAULT_DYNAMIC_SIZE)
        return tuple(out)

    def make_sample(self, dim_sizes: Optional[Dict[str, int]] = None) -> torch.Tensor:
        """A random tensor of this pattern; `dim_sizes` gives sizes for named dynamic dimensions."""
        shape = self.concrete_shape(dim_sizes)
        if self.dtype.is_floating_point:
            return torch.randn(shape, dtype=self.dtype)
        return torch.randint(0, 8, shape, dtype=self.dtype)

    def dynamic_dims(self, dim_pool: Optional[Dict[str, Any]] = None) -> Dict[int, Any]:
        """The `dynamic_shapes` entry torch.export wants for this input; `dim_pool` shares named symbols."""
        pool = dim_pool if dim_pool is not None else {}
        dims: Dict[int, Any] = {}
        for axis, d in enumerate(self.shape):
            if isinstance(d, int):
                continue
            if isinstance(d, str):
                dims[axis] = pool.setdefault(d, Dim(d))
            else:
                dims[axis] = Dim(f"_anon_{id(self)}_{axis}")
        return dims
