class PyMongoError(Exception): pass
class DuplicateKeyError(PyMongoError): pass
class BulkWriteError(PyMongoError): pass
