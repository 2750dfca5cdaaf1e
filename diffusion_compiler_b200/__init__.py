"""difb200: B200 (sm_100a) implementation of Diffusion Compiler's quantized DiT hot path.

``diffir``  DiffIR program model + DIFIR001 codec (host side)
``ops``     device-resident operators (ctypes into libdifb200.so, torch tensors as memory)
``build``   nvcc build of libdifb200.so
"""
__all__ = ["diffir", "ops", "build"]
