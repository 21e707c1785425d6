from .schedules import NoDecay  # import path kept for compatibility
