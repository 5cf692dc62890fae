from . import SCHEMA_PATH, write_schema

write_schema()
print(SCHEMA_PATH)
