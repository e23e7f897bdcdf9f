"""Engine-level facades: small, self-contained entry points over the trainers, the planners and the inference engine.

  dense      DenseTrainer, LRSchedule, OptimSuite, losses with explicit gradients, data loaders, DenseCheckpoint,
             UnifiedEntry, policy-gradient helpers, EvalHarness
  dense_extras  FinetuneRunner, LoRAEngine, QATEngine, MixedPrecision, ContinualRunner, EWCProbe
  multimodal    PatchEmbed, AudioFramer, VideoSampler, AlignTrainer, PerceiverTrainer, TokProbe, Sensor3D, FusionMath
  parallel   host-side planners and oracles: rank slices, ring all-reduce over per-rank vectors, TP splits, shard and
             pipeline plans
  moe        MoETrainerEngine, routing / capacity / expert-placement planners, dispatch-gather-combine oracles, MoEPipeline
  inference  text-in / text-out InferenceEngine facade with statistics and punctuation-buffered streaming

Reference counterparts: engines/trainer/dense/*, engines/trainer/moe/*, engines/inference/*."""
from . import dense, dense_extras, inference, moe, multimodal, parallel  # noqa: F401
