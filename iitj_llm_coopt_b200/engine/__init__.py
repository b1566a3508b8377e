from .context import GroupMeta, StepContext, Workspace
from .engine import Engine
from .llm import LLM, RequestOutput, build_engine
from .policy import StaticPolicy
from .runner import ModelRunner, StepEntry
from .scheduler import Plan, Scheduler, Sequence
