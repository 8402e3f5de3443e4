"""Typed configurations and the architecture-neutral model plan."""

from .model_plan import ConfigError, LayerSpec, ModelPlan, PartSpec, RunEntry, schedule_from_lists, sequential_schedule

__all__ = ["ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "RunEntry", "schedule_from_lists", "sequential_schedule"]
