def use_class_methods(*a, **k): pass
