class Database: pass
