"""humming_b200 -- B200 (sm_100a) native quantized GEMM behind Humming's layer API.

The public surface mirrors the reference project (inclusionAI/humming):
``humming_b200.dtypes`` (reference ``humming/dtypes.py``),
``humming_b200.layer.HummingLayer`` / ``HummingMethod`` / ``HummingLayerMeta``
(reference ``humming/layer.py``) and the generators in
``humming_b200.utils.test`` (reference ``humming/utils/test.py``);
``humming_b200.ops`` defines the reference's dispatcher operators
(``torch.ops.humming.launch_humming``, ``humming_quant_input``) and
``humming_b200.moe`` a whole MoE layer, single GPU or expert parallel.
All device work goes through the C ABI declared in ``include/humming_b200.h``;
there is no CPU fallback: importing :mod:`humming_b200.native` fails loudly if
the CUDA library has not been built.
"""

__version__ = "0.1.0"
