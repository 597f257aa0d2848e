"""Hand-written CUDA kernels for sm_100a (``*.cu``), their build (``build.py``) and their Python
bindings (``ops.py``)."""
