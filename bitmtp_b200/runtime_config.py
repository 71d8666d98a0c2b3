"""Runtime profiles; importing this module does not import PyTorch.

Mirrors `bonsai_sft.gpu.runtime_config` (src/bonsai_sft/gpu/runtime_config.py:8-67).
The reference's profiles choose between `torch.compile`d and eager helper
expressions; here every helper is a hand-written kernel, so a profile only
records the caller's choice and validates option combinations.  `b200` is the
default; the reference's names are accepted so existing command lines run.
"""
from __future__ import annotations

import sys
from typing import NamedTuple, Optional


class _Pinned(NamedTuple):
    """What an Orin profile of the reference fixes on the command line."""
    block_size: int
    ar_only: bool


# profile name -> pinned options (None: the profile admits every combination the CLI itself admits)
_TABLE = {
    'b200': None,
    'standard': None,
    'orin-sft': _Pinned(block_size=8, ar_only=True),
    'orin-d4': _Pinned(block_size=4, ar_only=False),
    'orin-d8': _Pinned(block_size=8, ar_only=False),
}
RUNTIME_PROFILES = tuple(_TABLE)
_RUNTIME_MODULES = ('model', 'fast_runtime', 'fast_generate')     # import these only after the profile is chosen
_profile = 'b200'


def _known(profile) -> str:
    if profile not in _TABLE:
        raise ValueError(f'unknown runtime profile: {profile}')
    return profile


def is_orin_profile(profile: Optional[str] = None) -> bool:
    name = _profile if profile is None else profile
    return name.startswith('orin-')


def current_profile() -> str:
    return _profile


def select_runtime_profile(profile) -> None:
    """Record the caller's profile.  As in the reference (runtime_config.py:15-25) a change of profile is refused
    once the runtime modules are imported, so that a command line cannot half-apply one."""
    global _profile
    _known(profile)
    if profile != _profile and any(f'{__package__}.{m}' in sys.modules for m in _RUNTIME_MODULES):
        raise RuntimeError('select the runtime profile before importing GPU runtime modules')
    _profile = profile


def compile_helper(fn=None, **kwargs):
    """Kept for source compatibility: helpers are never traced or compiled here."""
    if fn is None:
        return lambda function: function
    return fn


def validate_profile_options(args) -> None:
    """Option combinations a profile admits (src/bonsai_sft/gpu/runtime_config.py:36-55).

    The Orin profiles of the reference pin one block size, one mode family, native
    projections, a single 4096-token segment and the default threshold; the rules
    are kept so that a command line written for them is judged the same way.
    """
    name = _known(args.runtime_profile)
    pinned = _TABLE[name]
    if pinned is None:
        return
    native_heads = (args.draft_precision, args.verify_precision) == ('native', 'native')
    mode_rule = ((args.mode == 'ar', 'orin-sft requires AR mode') if pinned.ar_only
                 else (args.mode != 'ar', 'Orin MTP profiles require conf, spec, or hybrid mode'))
    rules = (
        (args.block_size == pinned.block_size, f'{name} requires block-size {pinned.block_size}'),
        mode_rule,
        (native_heads, 'Orin profiles require native T2 draft and verifier projections'),
        (args.max_context == 4096, 'Orin profiles require a single 4096-token segment'),
        (args.threshold == 0.9, 'Orin profiles require threshold 0.9'),
        (args.min_chain in (None, 3), 'Orin hybrid profiles require min-chain 3'),
    )
    for holds, message in rules:
        if not holds:
            raise ValueError(message)


def validate_profile_model(profile, config) -> None:
    if not is_orin_profile(profile):
        return
    geometry_ok = config.get('dim') == 2048 and config.get('kernel_kind') == 't2g128'
    if not geometry_ok:
        raise ValueError('Orin profiles support only Bonsai-1.7B native T2 checkpoints')


def validate_profile_device(profile, capability) -> None:
    if is_orin_profile(profile):
        raise ValueError('Orin profiles require an SM87 device; this build targets sm_100a')
