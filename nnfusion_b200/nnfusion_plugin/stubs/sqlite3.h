// Stand-in for sqlite3.h where SQLite's development files are not installed, for syntax checks of the plugin sources
// (src/nnfusion/engine/cache/manager.hpp holds a sqlite3* and nothing of the plugin calls into it).
#pragma once
struct sqlite3;
struct sqlite3_stmt;
