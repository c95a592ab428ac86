# Passed to the reference's unmodified CMake build through the CMAKE_TOOLCHAIN_FILE environment variable:
# tells FetchContent to use the third_party/ directories that are already populated (with the stand-ins
# of this folder) instead of cloning from the network.  Nothing else is changed.
set(FETCHCONTENT_FULLY_DISCONNECTED ON CACHE BOOL "use the populated third_party directories" FORCE)
# The reference relies on headers that older libstdc++ releases pulled in transitively (<mutex> for
# std::unique_lock in kraken/common/parallel_skip_list.h, <ctime> for time() in kraken/common/utils.h,
# ...); g++ 13 no longer does, so they are force-included here instead of editing the sources.
set(CMAKE_CXX_FLAGS_INIT "-include mutex -include ctime -include cstdint -include cstring -include functional -include stdexcept -include string -include limits -include memory -include algorithm")
# The reference links -lstdc++fs.  With g++ 13 std::filesystem lives in libstdc++.so and the static
# libstdc++fs.a carries private copies of locale internals; linked into a Python extension next to the
# process's libstdc++.so they crashed the first stream insertion inside kraken_native.initialize().
# The build script points this variable at a directory holding an EMPTY libstdc++fs.a, searched first.
if(DEFINED ENV{KRAKEN_BASELINE_LIBDIR})
  set(CMAKE_SHARED_LINKER_FLAGS_INIT "-L$ENV{KRAKEN_BASELINE_LIBDIR}")
  set(CMAKE_EXE_LINKER_FLAGS_INIT "-L$ENV{KRAKEN_BASELINE_LIBDIR}")
endif()
