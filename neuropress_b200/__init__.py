"""B200 (sm_100a) kernels for the forward of neuropress's lowered quantized linear layers.

Public surface, with the reference's names: ``neuropress_b200.nn`` (``NPVQLinear``, ``VQProxy``,
``NPLinear``, ``linearize_vq_weights``, ``linearize_qtensor_weights``, backend enums),
``neuropress_b200.kernel_lowering`` (``AutoKernelLowering``, ``LoweringConfig``, ``is_lowered``,
``unlower_model``), ``neuropress_b200.kernels`` (``vq_dequant``, ``vq_linear``,
``vq_linear_wmma``, ``q_linear`` ...), ``neuropress_b200.transforms.vq_packing.IndexPacking``.
The compute lives in ``libneuropress_b200.so`` (C ABI in ``include/neuropress_b200.h``), built
by ``python -m neuropress_b200.build``.
"""

from .kernel_lowering import AutoKernelLowering, LoweringConfig, is_lowered, unlower_model

__version__ = "0.1.0"
__all__ = ["AutoKernelLowering", "LoweringConfig", "is_lowered", "unlower_model", "__version__"]
