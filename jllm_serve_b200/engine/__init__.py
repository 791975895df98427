"""The engine: batch tables, the generic model, the step function, the scheduler and generation."""
from .batch import BatchBuilder, Segment, StepBatch
from .model import DecoderModel, build_model, model_wants
from .runner import ModelRunner
from .scheduler import Item, Pick, PlannedSegment, Request, Scheduler, plan_pass
from .engine import Engine, Result, Stats
