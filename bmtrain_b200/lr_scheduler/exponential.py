from .schedules import Exponential  # import path kept for compatibility
