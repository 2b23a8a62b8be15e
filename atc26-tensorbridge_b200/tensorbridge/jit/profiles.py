"""Measured `(max_m -> GemmConfig)` tables that override the selection rule per device, SM budget and weight shape.

Interface of the reference's `tensorbridge/jit/profiles.py:26-215`: `ProfileSegment`, `register_profile`,
`clear_profiles`, `load_profile_file`, `save_profile_file`, `lookup`, `compress_segments`.  A profile is keyed by
`(device name, SMs, padded n, padded k, experts, layout, group_scales, bridge)` and holds segments sorted by `max_m`;
the first segment with `m <= max_m` serves a call and `max_m == 0` marks an open-ended tail.

Files are JSON in the reference's schema, `{"schema_version": 1, "metadata": {...}, "entries": [{"device_name", "num_sms",
"n", "k", "num_experts", "layout", "group_scales", "bridge", "segments": [{"max_m", "config": [nine ints]}]}]}`; the
compact form this library's profile sweeper writes -- a bare list of entries with `"device"` and segments as
`[max_m, [nine ints]]` pairs -- loads as well.  Defaults come from `tensorbridge/profiles/*.json` and from every file or
directory on `TENSORBRIDGE_PROFILE_PATH` (separated like `PATH`), read on first use.
"""
from __future__ import annotations

import dataclasses
import json
import os
from collections.abc import Iterable, Sequence
from pathlib import Path

from tensorbridge.jit.codegen import Bridge, GemmConfig, GroupedLayout, pad_to_unit

PROFILES_DIR = Path(__file__).resolve().parent.parent / "profiles"
PROFILE_DIR = str(PROFILES_DIR)  # older name

ProfileKey = tuple[str, int, int, int, int, str, bool, str]


@dataclasses.dataclass(frozen=True)
class ProfileSegment:
    """Serves calls with `m <= max_m`; `max_m == 0` serves every larger m."""

    max_m: int
    config: GemmConfig


_registry: dict[ProfileKey, tuple[ProfileSegment, ...]] = {}
_defaults_loaded = False


def _key(device_name: str, num_sms: int, n: int, k: int, num_experts: int, layout: str, group_scales: bool, bridge: str) -> ProfileKey:
    return (str(device_name), int(num_sms), pad_to_unit(int(n)), pad_to_unit(int(k)), int(num_experts), str(layout),
            bool(group_scales), str(bridge))


def _ordered(segments: Iterable[ProfileSegment]) -> tuple[ProfileSegment, ...]:
    segments = list(segments)
    tails = [s for s in segments if s.max_m == 0]
    if len(tails) > 1:
        raise ValueError("a profile has at most one open-ended (max_m = 0) segment")
    return tuple(sorted((s for s in segments if s.max_m > 0), key=lambda s: s.max_m)) + tuple(tails)


def register_profile(device_name: str, num_sms: int, n: int, k: int, num_experts: int, layout: GroupedLayout,
                     group_scales: bool, bridge: Bridge, segments: Sequence[ProfileSegment]) -> None:
    """Add the profile of one shape and SM budget, replacing an earlier one with the same key."""
    _registry[_key(device_name, num_sms, n, k, num_experts, layout, group_scales, bridge)] = _ordered(segments)


def clear_profiles(*, reload_defaults: bool = False) -> None:
    """Forget every profile.  With `reload_defaults` the files on disk are read again at the next lookup; without it
    the registry stays empty until profiles are registered or loaded by hand."""
    global _defaults_loaded
    _registry.clear()
    _defaults_loaded = not reload_defaults


def reload() -> None:
    """Forget cached tables and read the default files again at the next lookup (after changing
    `TENSORBRIDGE_PROFILE_PATH` or writing a profile)."""
    clear_profiles(reload_defaults=True)


def _segments_of(entry: dict) -> list[ProfileSegment]:
    out = []
    for segment in entry["segments"]:
        if isinstance(segment, dict):
            max_m, values = segment["max_m"], segment["config"]
        else:
            max_m, values = segment
        out.append(ProfileSegment(int(max_m), GemmConfig.from_list(list(values))))
    return out


def load_profile_file(path: Path | str) -> int:
    """Register every entry of a profile JSON; returns how many."""
    data = json.loads(Path(path).read_text(encoding="utf-8"))
    entries = data["entries"] if isinstance(data, dict) else data
    for entry in entries:
        name = entry["device_name"] if "device_name" in entry else entry["device"]
        register_profile(name, entry["num_sms"], entry["n"], entry["k"], entry["num_experts"], entry["layout"],
                         entry["group_scales"], entry["bridge"], _segments_of(entry))
    return len(entries)


def save_profile_file(path: Path | str, entries: Sequence[tuple[ProfileKey, Sequence[ProfileSegment]]],
                      metadata: dict[str, object] | None = None) -> None:
    """Write `(key, segments)` pairs as a profile JSON in the canonical schema."""
    names = ("device_name", "num_sms", "n", "k", "num_experts", "layout", "group_scales", "bridge")
    payload = {"schema_version": 1, "metadata": metadata or {}, "entries": [
        dict(zip(names, key), segments=[{"max_m": s.max_m, "config": s.config.to_list()} for s in _ordered(segments)])
        for key, segments in entries]}
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(json.dumps(payload, indent=2) + "\n", encoding="utf-8")


def _load_defaults() -> None:
    global _defaults_loaded
    if _defaults_loaded:
        return
    _defaults_loaded = True
    sources = [PROFILES_DIR] + [Path(raw) for raw in os.environ.get("TENSORBRIDGE_PROFILE_PATH", "").split(os.pathsep) if raw]
    for source in sources:
        if source.is_dir():
            for file in sorted(source.glob("*.json")):
                load_profile_file(file)
        elif source.is_file():
            load_profile_file(source)


def lookup(device_name: str, num_sms: int, n: int, k: int, num_experts: int, layout: str, group_scales: bool, bridge: str,
           m: int) -> GemmConfig | None:
    """The profiled config for `m` rows of this shape, or None when no profile covers it (the rule decides then)."""
    _load_defaults()
    if not _registry:
        return None
    for segment in _registry.get(_key(device_name, num_sms, n, k, num_experts, layout, group_scales, bridge), ()):
        if segment.max_m == 0 or m <= segment.max_m:
            return segment.config
    return None


def compress_segments(points: Sequence[tuple[int, GemmConfig]], *, unbounded_tail: bool = False) -> list[ProfileSegment]:
    """`(m, winning config)` samples -> segments.  Neighbouring samples with one config merge; where the winner changes
    between two sampled m the boundary is their geometric mean (rounded down, never below the lower sample); the last
    segment ends at the last sample, or is open ended with `unbounded_tail`."""
    ordered = sorted(points, key=lambda point: point[0])
    segments: list[ProfileSegment] = []
    for index, (m, config) in enumerate(ordered):
        last = index == len(ordered) - 1
        if not last and ordered[index + 1][1] == config:
            continue
        if last:
            bound = 0 if unbounded_tail else m
        else:
            bound = max(m, int((m * ordered[index + 1][0]) ** 0.5))
        segments.append(ProfileSegment(bound, config))
    return segments
