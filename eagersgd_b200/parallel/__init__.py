"""Process group and partial allreduce backends."""
from .group import Group, init, finalize, rank, world_size  # noqa: F401
from ._native import ChannelError  # noqa: F401
from .partial_allreduce import PartialAllreduce  # noqa: F401
