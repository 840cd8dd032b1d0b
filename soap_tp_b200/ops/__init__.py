"""Composable distributed operations of the tensor-parallel SOAP pipeline.

The thirteen public names are those of the reference's ``soap_tp.ops``
(``src/soap_tp/ops/__init__.py:23-37``) with the same signatures.
"""
from ..layout import allocate_2d_block_cyclic
from .basis import (
    estimated_eigenvalue_order_2d_block_cyclic_,
    initialize_basis_2d_block_cyclic_,
    power_iteration_qr_2d_block_cyclic_,
    qr_2d_block_cyclic_,
    refresh_bases_and_transport_optimizer_state_,
)
from .elementwise import adam_update
from .gram import (
    update_left_preconditioner_2d_block_cyclic_,
    update_right_preconditioner_2d_block_cyclic_,
)
from .permute import permute_2d_block_cyclic_
from .redistribute import (
    redistribute_2d_block_cyclic_to_tp_shard,
    redistribute_tp_shard_to_2d_block_cyclic,
)
from .rotate import rotate_2d_block_cyclic_

__all__ = [
    "adam_update",
    "allocate_2d_block_cyclic",
    "estimated_eigenvalue_order_2d_block_cyclic_",
    "initialize_basis_2d_block_cyclic_",
    "permute_2d_block_cyclic_",
    "power_iteration_qr_2d_block_cyclic_",
    "qr_2d_block_cyclic_",
    "redistribute_2d_block_cyclic_to_tp_shard",
    "redistribute_tp_shard_to_2d_block_cyclic",
    "refresh_bases_and_transport_optimizer_state_",
    "rotate_2d_block_cyclic_",
    "update_left_preconditioner_2d_block_cyclic_",
    "update_right_preconditioner_2d_block_cyclic_",
]
