class CurriculumScheduler:
    """Sequence-length curriculum: fixed_linear schedule only."""

    def __init__(self, config):
        self.cfg = dict(config)
        self.min = config.get("min_difficulty", 1)
        self.max = config.get("max_difficulty", self.min)
        sc = config.get("schedule_config", {})
        self.total = sc.get("total_curriculum_step", 1)
        self.step_size = sc.get("difficulty_step", 1)
        self.current = self.min

    def get_current_difficulty(self):
        return self.current

    def update_difficulty(self, step):
        d = self.min + (self.max - self.min) * min(1.0, step / max(1, self.total))
        d = int(d) - int(d) % self.step_size
        self.current = max(self.min, min(self.max, d))
        return self.current
