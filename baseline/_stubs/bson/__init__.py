class ObjectId(str): pass
