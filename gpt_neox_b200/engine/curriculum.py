"""Sequence-length curriculum (DeepSpeed ``CurriculumScheduler`` used at ``megatron/training.py:1308-1311``).

Config block ``curriculum_learning``: ``min_difficulty``, ``max_difficulty``, ``schedule_type`` in
{``fixed_linear``, ``fixed_root``, ``fixed_discrete``} and ``schedule_config``."""
from __future__ import annotations

import math


class CurriculumScheduler:
    def __init__(self, config):
        self.state = {"min_difficulty": config["min_difficulty"], "max_difficulty": config["max_difficulty"],
                      "current_difficulty": config["min_difficulty"], "schedule_type": config["schedule_type"],
                      "schedule": dict(config.get("schedule_config", {}))}
        kind, sched = self.state["schedule_type"], self.state["schedule"]
        if kind == "fixed_discrete":
            assert len(sched["difficulty"]) == len(sched["max_step"]) + 1
        elif kind in ("fixed_linear", "fixed_root"):
            assert "total_curriculum_step" in sched and "difficulty_step" in sched
            if kind == "fixed_root":
                assert "root_degree" in sched
        else:
            raise RuntimeError(f"Unsupported curriculum schedule type {kind}")

    def get_current_difficulty(self):
        return self.state["current_difficulty"]

    def set_current_difficulty(self, d):
        self.state["current_difficulty"] = d

    def get_state(self):
        return self.state

    def set_state(self, s):
        self.state = s

    def _root(self, step, degree):
        s = self.state["schedule"]
        frac = (float(step) / s["total_curriculum_step"]) ** (1.0 / degree)
        d = math.floor(frac * (self.state["max_difficulty"] - self.state["min_difficulty"]) + self.state["min_difficulty"])
        d -= d % s["difficulty_step"]
        return min(d, self.state["max_difficulty"])

    def get_difficulty(self, step):
        kind, s = self.state["schedule_type"], self.state["schedule"]
        if kind == "fixed_discrete":
            if step > s["max_step"][-1]:
                return s["difficulty"][-1]
            for i, m in enumerate(s["max_step"]):
                if step <= m:
                    return s["difficulty"][i]
        if kind == "fixed_linear":
            return self._root(step, 1)
        return self._root(step, s["root_degree"])

    def update_difficulty(self, step):
        if self.state["current_difficulty"] < self.state["max_difficulty"]:
            self.state["current_difficulty"] = self.get_difficulty(step)
        return self.state["current_difficulty"]
