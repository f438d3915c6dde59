"""Stand-in: the benchmark arm never opens a database."""
from . import database, errors, results  # noqa: F401

ASCENDING = 1
DESCENDING = -1


class MongoClient:
    def __init__(self, *a, **k):
        raise RuntimeError("pymongo is not installed")


class UpdateOne:
    def __init__(self, *a, **k):
        raise RuntimeError("pymongo is not installed")
