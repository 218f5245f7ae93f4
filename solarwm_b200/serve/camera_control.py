"""Keyboard camera control: discrete key states -> smooth absolute camera trajectory.

The model is conditioned on poses, never on key symbols.  ``w a s d`` translate (forward / left /
back / right), ``i k`` pitch, ``j l`` yaw.  A state advanced once per output video frame holds a
local linear velocity and pitch / yaw rates that move towards their key-selected targets with a
bounded acceleration; the pose is integrated as ``R' = Ry(yaw) R Rx(pitch)`` (pitch clamped) and
``t' = t + R' v dt`` (optionally constrained to the ground plane).  Action strings such as
``w-3,wl-2,none-1`` give one key set per latent interval; each latent interval spans
``temporal_stride`` pixel frames, and the per-latent camera-to-world matrices handed to the model are
sampled at the latent-aligned pixel indices (0, 1, 5, 9, ...).

Reference: deploy/solar_wm/shared/runtime/camera.py:39-509, navigation.py:13-106.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

import numpy as np

ALLOWED_KEYS = frozenset("wasdijkl")
_ORDER = "wasdijkl"
MIN_MOVE_SCALE, MAX_MOVE_SCALE = 0.25, 4.0


def normalize_keys(keys: Iterable[str]) -> List[str]:
    if isinstance(keys, str):
        keys = list(keys)
    got = {str(k).lower() for k in keys}
    bad = sorted(got - ALLOWED_KEYS)
    if bad:
        raise ValueError(f"invalid camera key(s) {bad!r}; allowed keys are w,a,s,d,i,j,k,l")
    return [k for k in _ORDER if k in got]


def parse_action_string(text: str) -> List[List[str]]:
    """``w-3,wl-2,none-1`` -> one key list per latent interval."""
    if not isinstance(text, str):
        raise TypeError("action_string must be a string")
    flat = "".join(text.replace("，", ",").split())
    if not flat:
        raise ValueError("action_string is empty")
    out: List[List[str]] = []
    for seg in flat.split(","):
        if not seg:
            raise ValueError("action_string has an empty segment (check commas)")
        if "-" not in seg:
            raise ValueError(f"invalid segment {seg!r}: expected <keys>-<duration>")
        keys_text, dur = seg.rsplit("-", 1)
        if not dur.isdigit() or int(dur) <= 0:
            raise ValueError(f"invalid duration in segment {seg!r}: expected a positive integer")
        keys_text = keys_text.lower()
        if keys_text == "none":
            keys: List[str] = []
        elif not keys_text:
            raise ValueError(f"invalid segment {seg!r}: use 'none' for a neutral step")
        else:
            keys = normalize_keys(keys_text)
        out.extend([list(keys) for _ in range(int(dur))])
    return out


def fit_action_steps(actions: Sequence[Sequence[str]], *, num_transitions: int) -> List[List[str]]:
    if num_transitions < 0:
        raise ValueError("num_transitions must be non-negative")
    norm = [normalize_keys(a) for a in actions]
    if len(norm) > num_transitions:
        raise ValueError(f"action schedule has {len(norm)} transitions, but the rollout only has room for {num_transitions}")
    return norm + [[] for _ in range(num_transitions - len(norm))]


def _rot(axis: str, angle: float) -> np.ndarray:
    c, s = math.cos(angle), math.sin(angle)
    if axis == "x":
        return np.array([[1, 0, 0], [0, c, -s], [0, s, c]], dtype=np.float64)
    if axis == "y":
        return np.array([[c, 0, s], [0, 1, 0], [-s, 0, c]], dtype=np.float64)
    raise ValueError(axis)


def _towards(cur, target, max_delta):
    cur, target = np.asarray(cur, dtype=np.float64), np.asarray(target, dtype=np.float64)
    diff = target - cur
    dist = float(np.linalg.norm(diff))
    if dist <= max_delta or dist == 0.0:
        return target.copy()
    return cur + diff * (max_delta / dist)


@dataclass(frozen=True)
class KeyboardCameraConfig:
    frames_per_second: float = 16.0
    move_speed_per_second: float = 1.2
    pitch_speed_degrees_per_second: float = 24.0
    yaw_speed_degrees_per_second: float = 24.0
    acceleration_seconds: float = 0.25
    pitch_limit_degrees: float = 85.0
    ground_plane_translation: bool = False

    def __post_init__(self):
        vals = (self.frames_per_second, self.move_speed_per_second, self.pitch_speed_degrees_per_second,
                self.yaw_speed_degrees_per_second, self.acceleration_seconds, self.pitch_limit_degrees)
        if not all(math.isfinite(float(v)) for v in vals):
            raise ValueError("keyboard camera configuration must be finite")
        if self.frames_per_second <= 0:
            raise ValueError("frames_per_second must be positive")
        if min(self.move_speed_per_second, self.pitch_speed_degrees_per_second, self.yaw_speed_degrees_per_second,
               self.acceleration_seconds) < 0:
            raise ValueError("speeds and acceleration time must be non-negative")
        if not 0 < self.pitch_limit_degrees < 90:
            raise ValueError("pitch_limit_degrees must be in (0, 90)")


class KeyboardCameraState:
    def __init__(self, config: Optional[KeyboardCameraConfig] = None, *, initial_c2w=None, move_speed_scale: float = 1.0):
        self.config = config or KeyboardCameraConfig()
        self.c2w = np.eye(4, dtype=np.float64) if initial_c2w is None else np.asarray(initial_c2w, dtype=np.float64).copy()
        self.velocity = np.zeros(3)
        self.pitch_rate = 0.0
        self.yaw_rate = 0.0
        self.pitch = 0.0
        self.set_move_speed_scale(move_speed_scale)

    def set_move_speed_scale(self, value: float = 1.0) -> float:
        if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)) or \
                not MIN_MOVE_SCALE <= float(value) <= MAX_MOVE_SCALE:
            raise ValueError("move_speed_scale must be a finite number from 0.25 to 4.0")
        self.move_scale = float(value)
        return self.move_scale

    def step(self, keys: Iterable[str]) -> np.ndarray:
        """Advance one output video frame; returns the new camera-to-world matrix (fp32)."""
        k = normalize_keys(keys)
        cfg = self.config
        dt = 1.0 / cfg.frames_per_second
        speed = cfg.move_speed_per_second * self.move_scale
        tv = np.array([speed * (("d" in k) - ("a" in k)), 0.0, speed * (("w" in k) - ("s" in k))])
        tp = cfg.pitch_speed_degrees_per_second * (("i" in k) - ("k" in k))
        ty = cfg.yaw_speed_degrees_per_second * (("l" in k) - ("j" in k))
        if cfg.acceleration_seconds == 0:
            self.velocity, self.pitch_rate, self.yaw_rate = tv, float(tp), float(ty)
        else:
            a = dt / cfg.acceleration_seconds
            self.velocity = _towards(self.velocity, tv, speed * a)
            self.pitch_rate = float(_towards([self.pitch_rate], [tp], cfg.pitch_speed_degrees_per_second * a)[0])
            self.yaw_rate = float(_towards([self.yaw_rate], [ty], cfg.yaw_speed_degrees_per_second * a)[0])
        dp, dy = math.radians(self.pitch_rate * dt), math.radians(self.yaw_rate * dt)
        lim = math.radians(cfg.pitch_limit_degrees)
        if self.pitch + dp > lim:
            dp, self.pitch, self.pitch_rate = lim - self.pitch, lim, 0.0
        elif self.pitch + dp < -lim:
            dp, self.pitch, self.pitch_rate = -lim - self.pitch, -lim, 0.0
        else:
            self.pitch += dp
        R = _rot("y", dy) @ self.c2w[:3, :3] @ _rot("x", dp)
        if cfg.ground_plane_translation:
            fwd, right = R[:, 2].copy(), R[:, 0].copy()
            fwd[1] = right[1] = 0.0
            for vec in (fwd, right):
                n = float(np.linalg.norm(vec))
                if n:
                    vec /= n
            world_v = right * self.velocity[0] + fwd * self.velocity[2]
        else:
            world_v = R @ self.velocity
        out = np.eye(4)
        out[:3, :3] = R
        out[:3, 3] = self.c2w[:3, 3] + world_v * dt
        self.c2w = out
        return out.astype(np.float32)


def actions_to_latent_c2w(actions: Sequence[Sequence[str]], *, temporal_stride: int = 4,
                          config: Optional[KeyboardCameraConfig] = None, state: Optional[KeyboardCameraState] = None,
                          include_first: bool = True) -> np.ndarray:
    """One camera-to-world matrix per latent frame: the starting pose (optional) then the pose after
    each latent interval of ``temporal_stride`` pixel frames."""
    st = state or KeyboardCameraState(config)
    poses = [st.c2w.astype(np.float32)] if include_first else []
    for keys in actions:
        for _ in range(temporal_stride):
            pose = st.step(keys)
        poses.append(pose)
    return np.stack(poses) if poses else np.zeros((0, 4, 4), dtype=np.float32)


class NavigationState:
    """Live key state of an interactive session: keys held down, speed scales, pause."""

    def __init__(self, config: Optional[KeyboardCameraConfig] = None):
        self.camera = KeyboardCameraState(config)
        self.down: set = set()
        self.turn_scale = 1.0
        self.paused = False

    def set_key(self, key: str, down: bool) -> None:
        key = normalize_keys([key])[0]
        (self.down.add if down else self.down.discard)(key)

    def set_speeds(self, move: float, turn: float) -> None:
        self.camera.set_move_speed_scale(min(max(float(move), MIN_MOVE_SCALE), MAX_MOVE_SCALE))
        self.turn_scale = min(max(float(turn), 0.1), 3.0)

    def next_actions(self, count: int) -> List[List[str]]:
        keys = [] if self.paused else normalize_keys(self.down)
        return [list(keys) for _ in range(count)]

    def advance(self, latent_frames: int, temporal_stride: int = 4) -> np.ndarray:
        return actions_to_latent_c2w(self.next_actions(latent_frames), temporal_stride=temporal_stride,
                                     state=self.camera, include_first=False)
