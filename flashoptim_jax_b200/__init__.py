"""flashoptim_jax_b200: the optimizer-step hot path of flashoptim-jax as sm_100a CUDA kernels.

The exported names are those of the reference package (flashoptim_jax/__init__.py:31-57);
arrays are CUDA torch tensors and every computation is a call into libflashoptim_b200.so.
"""

from .adamw import FlashAdamState, flash_adam, flash_adamw, flash_adamw_state_dict, load_flash_adamw_state_dict
from .compression import cast_tree_bf16, reconstruct_leaf, reconstruct_weights, set_fp32_params, split_leaf
from .lion import FlashLionState, flash_lion, flash_lion_state_dict, load_flash_lion_state_dict
from .quantization import QuantizedArray, dequantize_momentum, dequantize_variance, quantize_momentum, quantize_variance
from .sgd import FlashSGDState, flash_sgd, flash_sgd_state_dict, flash_sgdw, load_flash_sgd_state_dict
from .utils import FlashOptimizer

__all__ = [
    "FlashAdamState", "FlashOptimizer", "FlashLionState", "FlashSGDState", "QuantizedArray", "cast_tree_bf16",
    "dequantize_momentum", "dequantize_variance", "flash_adam", "flash_adamw", "flash_lion", "flash_lion_state_dict",
    "flash_sgd", "flash_sgd_state_dict", "flash_sgdw", "flash_adamw_state_dict", "load_flash_adamw_state_dict",
    "load_flash_lion_state_dict", "load_flash_sgd_state_dict", "quantize_momentum", "quantize_variance",
    "reconstruct_leaf", "reconstruct_weights", "set_fp32_params", "split_leaf",
]
