"""Offline density profile lookup (Step,Layer,Head,Sparsity CSV); interface of the
reference's svoo/sparsity/lookup.py:9-45 plus the per-head clipping of
svoo/models/wan/attention.py:931-956."""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union


class SparsityLookup:
    """In-memory table of per-(step, layer, head) key-cluster density."""

    def __init__(self, csv_path: str):
        self.lookup_dict: Dict[Tuple[int, int, int], float] = {}
        self._load_csv(csv_path)

    def _load_csv(self, csv_path: str) -> None:
        f = Path(csv_path)
        if not f.exists():
            raise FileNotFoundError(f"Sparsity CSV file not found: {csv_path}")
        with open(f, "r", encoding="utf-8") as fh:
            for row in csv.DictReader(fh):
                self.lookup_dict[(int(row["Step"]), int(row["Layer"]), int(row["Head"]))] = float(row["Sparsity"])

    def get_sparsity(self, step: int, layer: int, head: int) -> Optional[float]:
        return self.lookup_dict.get((step, layer, head))

    def get_sparsity_batch(self, step: int, layer: int, num_heads: int) -> List[float]:
        return [self.get_sparsity(step, layer, h) or 0.0 for h in range(num_heads)]

    def has_data_for_step_layer(self, step: int, layer: int, num_heads: int = 12) -> bool:
        return all(self.get_sparsity(step, layer, h) is not None for h in range(num_heads))


def min_kc_ratio_for_heads(lookup: Optional[SparsityLookup], use_dynamic: bool, step: Optional[int], layer: int,
                           num_heads: int, fallback, lo: Optional[float], hi: Optional[float]
                           ) -> Union[float, List[float]]:
    """Per-head floor ratios clipped to [lo, hi], or `fallback` when the table has no
    complete entry for (step, layer) (svoo/models/wan/attention.py:931-956)."""
    if use_dynamic and lookup is not None and step is not None:
        if not lookup.has_data_for_step_layer(step, layer, num_heads):
            return fallback
        out = []
        for v in lookup.get_sparsity_batch(step, layer, num_heads):
            if lo is not None:
                v = max(v, lo)
            if hi is not None:
                v = min(v, hi)
            out.append(v)
        return out
    return fallback
