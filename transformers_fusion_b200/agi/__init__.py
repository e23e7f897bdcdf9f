"""Self-monitoring, planning, multi-agent and evaluation scaffolding around a text model.

Everything here talks to the model through two small callables, so that it works with the inference engine, a server
client or a stub in tests: ``generate(prompt) -> str`` and (where probabilities matter) ``logits(prompt) -> Tensor[V]``.

Reference counterparts: include/quant/agi.h (SelfMonitor :111 ... Flywheel :473), meta_cognition.h, multi_agent.h,
self_eval.h, world_model.h; src/agi/*.cpp."""
from .core import (HITL, AlertEntry, AlignmentSystem, AuditEntry, ChainOfThought, ContinuousLearner, CuriosityDrivenExplorer,  # noqa: F401
                   EvaluationHarness, Flywheel, KnowledgeDistillation, MemorySystem, Message, MetaCognition, MetaCognitionState,
                   MultiAgentCoordinator, PlanningEngine, PlanStep, PromptOptimizer, RecursiveSelfImprover, RollingStats,
                   SafetyGuardrails, Sandbox, SandboxResult, SelfMonitor, SelfReflector, SelfVerifier, ToolUse)
from .meta import MetaCognitionEngine  # noqa: F401
from .multi_agent import MultiAgentSystem  # noqa: F401
from .self_eval import SelfEvalSuite, pass_at_k  # noqa: F401
from .world_model import WorldModel  # noqa: F401
