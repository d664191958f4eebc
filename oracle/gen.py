"""Seeded inputs for the parity tests: the generators live with the product
(mongoose_b200/synthetic.py, the benchmark needs them too) and are re-exported
here so that tests read ``from oracle import gen``."""
from mongoose_b200.synthetic import (model_slots, norm_vector, prompt_ids,  # noqa: F401
                                     single_matvec_case, tensor_f32)
