from .warmup import WarmupLRScheduler
from .schedules import NoDecay, Noam, Linear, Cosine, Exponential
