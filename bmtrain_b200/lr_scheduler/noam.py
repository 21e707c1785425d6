from .schedules import Noam  # import path kept for compatibility
