"""Trajectory IO is outside the hot path this package replaces; the names exist so that callers
import, and using them says where to get the real ones."""

import os

_MSG = "trajectory IO is not part of dynamis_b200: use the reference's dynamis_state.io for it"


def is_pathlike(obj) -> bool:
    return isinstance(obj, (str, bytes, os.PathLike))


class TrajectoryReader:
    def __init__(self, *a, **k):
        raise NotImplementedError(_MSG)


class TrajectoryWriter:
    def __init__(self, *a, **k):
        raise NotImplementedError(_MSG)


def translate_dynamis_to_xyz(*a, **k):
    raise NotImplementedError(_MSG)
