from lily_b200.parts.base import (Block, BlockSpec, BuildContext, CacheNeed, FeedForward, Mixer, ModelSpec, Norm,
                                  Part, ScheduleEntry, StateNeed, TensorSpec, build_part, register_part, registered)

__all__ = ["Block", "BlockSpec", "BuildContext", "CacheNeed", "FeedForward", "Mixer", "ModelSpec", "Norm", "Part",
           "ScheduleEntry", "StateNeed", "TensorSpec", "build_part", "register_part", "registered"]
