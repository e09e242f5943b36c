"""Torch-facing operators backed by the sm_100a kernels."""
