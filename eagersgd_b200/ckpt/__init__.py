"""Checkpointing: tf-models variable layout, per-rank directories, rank-0 re-sync."""
from .tf_layout import (tf_variables, export_tf_layout, import_tf_layout, save, load, latest, clean,  # noqa: F401
                        resync_from_rank0)
