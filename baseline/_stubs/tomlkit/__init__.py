def parse(s):
    import tomllib

    return tomllib.loads(s)


loads = parse
