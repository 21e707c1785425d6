from .schedules import Cosine  # import path kept for compatibility
