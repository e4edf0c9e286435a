"""Drop-in name of the reference's extension module (`fp6_llm_cuda`, setup.py:34 and fp6_llm/csrc/pybind.cpp:6-16 of
usyd-fsalab/fp6_llm): the six functions the reference binds, backed by libfp6_b200.so through fp6_llm_b200.  Like
the pybind functions they take positional arguments only in the reference; keyword use is not part of the contract."""
from fp6_llm_b200 import (linear_forward_cuda, linear_forward_eXmY_cuda, weight_dequant_cpu, weight_dequant_eXmY_cpu,
                          weight_prepacking_cpu, weight_prepacking_eXmY_cpu)

__all__ = ["linear_forward_cuda", "weight_prepacking_cpu", "weight_dequant_cpu", "linear_forward_eXmY_cuda",
           "weight_prepacking_eXmY_cpu", "weight_dequant_eXmY_cpu"]
