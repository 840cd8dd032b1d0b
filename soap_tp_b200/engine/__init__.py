"""CUDA (sm_100a) engine: Python drivers of the native kernels in ``soap_tp_b200/csrc``."""
