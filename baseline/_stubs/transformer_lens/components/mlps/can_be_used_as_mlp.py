class CanBeUsedAsMLP:  # placeholder
    pass
