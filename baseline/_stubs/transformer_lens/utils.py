class Slice:  # placeholder
    pass


SliceInput = object
