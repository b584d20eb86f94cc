"""B200 (sm_100a) implementation of the UMA-QMoE routed-expert operator.

Public names follow the reference package (``uma_qmoe.custom_op`` and
``uma_qmoe.native_backend``) so a host written against it switches by import.
"""

from .custom_op import (PLATFORM, acquire_expert_pack, expert_pack_for_handle, register_expert_pack,
                        register_moe_forward, register_performance_backend, register_target_pack,
                        unregister_expert_pack)
from .formats import ContractError
from .pack_files import ExpertPackFile, TargetPackFile

__all__ = [
    "PLATFORM", "ContractError", "acquire_expert_pack", "expert_pack_for_handle", "register_expert_pack",
    "register_moe_forward", "register_performance_backend", "register_target_pack", "unregister_expert_pack",
    "install_packed_q4_backend", "install_mixed_target_backend", "ExpertPackFile", "TargetPackFile",
]


def install_packed_q4_backend(**kwargs):
    from .native_backend import install_packed_q4_backend as f
    return f(**kwargs)


def install_mixed_target_backend(**kwargs):
    from .native_backend import install_mixed_target_backend as f
    return f(**kwargs)
