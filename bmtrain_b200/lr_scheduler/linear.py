from .schedules import Linear  # import path kept for compatibility
