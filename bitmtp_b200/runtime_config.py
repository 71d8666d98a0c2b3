"""Runtime profiles; importing this module does not import PyTorch.

Mirrors `bonsai_sft.gpu.runtime_config` (src/bonsai_sft/gpu/runtime_config.py:8-67).
The reference's profiles choose between `torch.compile`d and eager helper
expressions; here every helper is a hand-written kernel, so a profile only
records the caller's choice and validates option combinations.  `b200` is the
default; the reference's names are accepted so existing command lines run.
"""
from __future__ import annotations

import sys

RUNTIME_PROFILES = ('b200', 'standard', 'orin-sft', 'orin-d4', 'orin-d8')
_profile = 'b200'


def is_orin_profile(profile=None):
    return (profile if profile is not None else _profile).startswith('orin-')


def current_profile() -> str:
    return _profile


def select_runtime_profile(profile):
    """Select before importing model/atlas helpers (runtime_config.py:15-25)."""
    global _profile
    if profile not in RUNTIME_PROFILES:
        raise ValueError(f'unknown runtime profile: {profile}')
    loaded = any(f'bitmtp_b200.{name}' in sys.modules
                 for name in ('model', 'fast_runtime', 'fast_generate'))
    if loaded and profile != _profile:
        raise RuntimeError('select the runtime profile before importing GPU runtime modules')
    _profile = profile


def compile_helper(fn=None, **kwargs):
    """Kept for source compatibility: helpers are never traced or compiled here."""
    return fn if fn is not None else (lambda function: function)


def validate_profile_options(args):
    """Option combinations a profile admits (src/bonsai_sft/gpu/runtime_config.py:36-55).

    The Orin profiles of the reference pin one block size, one mode family, native
    projections, a single 4096-token segment and the default threshold; the rules
    are kept so that a command line written for them is judged the same way.
    """
    profile = args.runtime_profile
    if profile not in RUNTIME_PROFILES:
        raise ValueError(f'unknown runtime profile: {profile}')
    if not is_orin_profile(profile):
        return
    want_block = {'orin-d4': 4}.get(profile, 8)
    sft = profile == 'orin-sft'
    rules = (
        (args.block_size == want_block, f'{profile} requires block-size {want_block}'),
        (not sft or args.mode == 'ar', 'orin-sft requires AR mode'),
        (sft or args.mode != 'ar', 'Orin MTP profiles require conf, spec, or hybrid mode'),
        (args.draft_precision == 'native' and args.verify_precision == 'native',
         'Orin profiles require native T2 draft and verifier projections'),
        (args.max_context == 4096, 'Orin profiles require a single 4096-token segment'),
        (args.threshold == 0.9, 'Orin profiles require threshold 0.9'),
        (args.min_chain in (None, 3), 'Orin hybrid profiles require min-chain 3'),
    )
    for ok, message in rules:
        if not ok:
            raise ValueError(message)


def validate_profile_model(profile, config):
    if is_orin_profile(profile) and (config.get('dim') != 2048
                                     or config.get('kernel_kind') != 't2g128'):
        raise ValueError('Orin profiles support only Bonsai-1.7B native T2 checkpoints')


def validate_profile_device(profile, capability):
    if is_orin_profile(profile):
        raise ValueError('Orin profiles require an SM87 device; this build targets sm_100a')
