"""soap_tp_b200: tensor-parallel SOAP for NVIDIA B200 (sm_100a).

Public surface mirrors the reference package (``src/soap_tp/__init__.py:1-4``): ``soap_step``
and the ``ops`` namespace; added on top are the ``SoapTP`` optimizer wrapper, the Llama-shaped
tensor-parallel model and the communicator.
"""
from . import ops
from .step import soap_step

__version__ = "0.1.0"


def __getattr__(name):
    if name == "SoapTP":
        from .optim import SoapTP

        return SoapTP
    raise AttributeError(name)


__all__ = ["SoapTP", "ops", "soap_step"]
