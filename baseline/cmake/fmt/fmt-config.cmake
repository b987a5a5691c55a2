# Header-only `fmt::fmt` for an offline build of the reference: the fmt headers that ship
# inside the installed torch wheel (torch/include/fmt), consumed with FMT_HEADER_ONLY.
# FMT_INCLUDE_DIR is passed on the cmake command line by build_reference.py.
if(NOT TARGET fmt::fmt)
  add_library(fmt::fmt INTERFACE IMPORTED)
  set_target_properties(fmt::fmt PROPERTIES
    INTERFACE_INCLUDE_DIRECTORIES "${FMT_INCLUDE_DIR}"
    INTERFACE_COMPILE_DEFINITIONS "FMT_HEADER_ONLY=1")
endif()
set(fmt_FOUND TRUE)
set(fmt_VERSION 12.1.0)
