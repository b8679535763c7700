"""Kernel backends: the operator surface of the EXL3 linear and MoE layers on B200."""
