"""Mask compiler and attention kernels; thin aliases of ``systems_for_llms_b200.attention``."""
