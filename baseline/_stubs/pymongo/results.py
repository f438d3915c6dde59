class UpdateResult: pass
class InsertOneResult: pass
class DeleteResult: pass
class BulkWriteResult: pass
