"""Drop-in module name of the reference package (fp6_llm/__init__.py:1-23 of usyd-fsalab/fp6_llm): `import fp6_llm`
gives the same six operators, `Num_Wave` and `HeuristicFuntion_SplitK`, implemented by fp6_llm_b200 for B200."""
from fp6_llm_b200 import (HeuristicFuntion_SplitK, Num_Wave, linear_forward_cuda, linear_forward_eXmY_cuda,
                          weight_dequant_cpu, weight_dequant_eXmY_cpu, weight_prepacking_cpu, weight_prepacking_eXmY_cpu)

__all__ = ["linear_forward_cuda", "weight_prepacking_cpu", "weight_dequant_cpu", "linear_forward_eXmY_cuda",
           "weight_prepacking_eXmY_cpu", "weight_dequant_eXmY_cpu", "Num_Wave", "HeuristicFuntion_SplitK"]
