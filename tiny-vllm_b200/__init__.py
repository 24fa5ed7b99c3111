"""B200 (sm_100a) implementation of tiny-vLLM's quantized linear path.

Sub-packages mirror the reference's module layout for this path:

* ``quantization`` — ``QuantMethod`` plug-ins (W8A16, W8A8) and the functions
  that call the CUDA library (reference: ``nanovllm/quantization``).
* ``layers.linear`` — tensor-parallel linear layers with the reference's
  constructors and weight loaders (reference: ``nanovllm/layers/linear.py``).
* ``utils.loader`` — safetensors loader for plain and quantized artifacts
  (reference: ``nanovllm/utils/loader.py``).
* ``_lib`` — ctypes binding of ``libb200q.so`` (C ABI in ``include/b200q.h``).
"""

__version__ = "0.1.0"
