"""`import fp6_llm` and `import fp6_llm_cuda` (the reference's module names, fp6_llm/__init__.py:1 and setup.py:34)
resolve to this library's operators."""


def test_reference_module_names_export_the_reference_functions():
    import fp6_llm
    import fp6_llm_b200
    import fp6_llm_cuda
    six = ("linear_forward_cuda", "weight_prepacking_cpu", "weight_dequant_cpu", "linear_forward_eXmY_cuda",
           "weight_prepacking_eXmY_cpu", "weight_dequant_eXmY_cpu")
    for name in six:
        assert getattr(fp6_llm_cuda, name) is getattr(fp6_llm_b200, name)
        assert getattr(fp6_llm, name) is getattr(fp6_llm_b200, name)
    # the pure-Python heuristic keeps the reference's spelling and values (fp6_llm/__init__.py:6-23)
    assert fp6_llm.HeuristicFuntion_SplitK(4096, 8, 108) == fp6_llm_b200.HeuristicFuntion_SplitK(4096, 8, 108)
    assert abs(fp6_llm.Num_Wave(4096, 8, 3, 108) - 8 * 1 * 3 / 108) < 1e-12
