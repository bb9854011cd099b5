"""Import path of the optimisation switches and variant names in the reference package
(qwen3_triton/configuration.py there); they are defined with the graph in qwen3_triton/_model.py."""
from ._model import ABLATIONS, VARIANTS, ComputeOptions, OptimizationOptions, options_for_variant  # noqa: F401
