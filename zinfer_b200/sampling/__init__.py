from .sampler import Sampler, SamplingParams, dry_penalties, recent_distinct, uniform
