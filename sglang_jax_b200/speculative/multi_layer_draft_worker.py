"""NEXTN / MTP drafting with one or more prediction layers.

Draft step `s` runs MTP layer `min(s, n_layers - 1)`; the passes that populate the draft
caches (after prefill and after verification) run every layer so that each layer's KV
covers the accepted prefix.  With a single MTP layer this reduces to the EAGLE chain.

Reference: `python/sgl_jax/srt/speculative/multi_layer_draft_worker.py`.
"""

from __future__ import annotations

from .base_worker import SpecInput
from .eagle_draft_worker import EagleDraftWorker


class MultiLayerDraftWorker(EagleDraftWorker):
    def __init__(self, server_args, target_worker, algo, owner):
        super().__init__(server_args, target_worker, algo, owner)
        self.num_mtp_layers = int(getattr(self.model, "num_mtp_layers", 1))
        self.uses_hidden = True

    def decorate_spec(self, spec: SpecInput, step: int | None) -> SpecInput:
        if step is None:
            spec.mtp_all_layers = self.num_mtp_layers > 1
        else:
            spec.mtp_layer = min(step, self.num_mtp_layers - 1)
        return spec
