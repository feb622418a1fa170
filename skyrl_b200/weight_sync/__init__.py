"""Trainer -> rollout-engine weight synchronisation."""

from .base import LoraLoadRequest, WeightChunk, WeightExtractor, WeightUpdateRequest
from .extractor import FlatModelWeightExtractor
from .strategies import (BroadcastStrategy, InPlaceStrategy, PeerPushStrategy, WeightTransferStrategy,
                         load_chunk_into_model, select_strategy_name)

__all__ = ["WeightChunk", "WeightUpdateRequest", "LoraLoadRequest", "WeightExtractor", "FlatModelWeightExtractor",
           "WeightTransferStrategy", "InPlaceStrategy", "PeerPushStrategy", "BroadcastStrategy", "load_chunk_into_model",
           "select_strategy_name"]
