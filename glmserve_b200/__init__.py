"""glmserve_b200: the W4A16 MoE layer path of glmserve, written for B200 (sm_100a).

``glmserve_b200.ops`` mirrors the reference's operator surface on top of the C ABI in
``include/glmserve_b200.h``; ``glmserve_b200.synth`` / ``quant`` build seeded synthetic
layers in the reference's weight layout.  Importing the package does not load CUDA.
"""
__all__ = ["ops", "quant", "synth", "build"]
