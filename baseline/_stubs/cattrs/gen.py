def make_dict_structure_fn(*a, **k):
    return lambda *x, **y: (_ for _ in ()).throw(RuntimeError("cattrs is not installed"))


def make_dict_unstructure_fn(*a, **k):
    return lambda *x, **y: (_ for _ in ()).throw(RuntimeError("cattrs is not installed"))


def override(*a, **k):
    return None
