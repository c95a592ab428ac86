// The reference includes this header (kraken/ps/sparse_table.h:9) but uses nothing from it.
#pragma once
