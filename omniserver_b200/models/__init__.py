"""Model specs and the executor that runs them."""

from .decoder import DecoderModel, EntryNeeds
from .spec import LayerSpec, ModelSpec, ScheduleEntry
from . import qwen2_vl  # noqa: F401  (registers the architecture)
