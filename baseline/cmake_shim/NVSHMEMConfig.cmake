# CMake package shim for the pip wheel nvidia-nvshmem-cu12, which ships headers and libraries
# but no CMake package.  Provides the two imported targets the reference links against.
execute_process(
  COMMAND python -c "import os, nvidia; print(os.path.join(os.path.dirname(nvidia.__path__[0]), 'nvidia', 'nvshmem'))"
  OUTPUT_VARIABLE NVSHMEM_ROOT OUTPUT_STRIP_TRAILING_WHITESPACE)
if(NOT EXISTS "${NVSHMEM_ROOT}/include/nvshmem.h")
  message(FATAL_ERROR "nvidia-nvshmem-cu12 not found under ${NVSHMEM_ROOT}")
endif()
find_package(CUDAToolkit REQUIRED)
if(NOT TARGET nvshmem::nvshmem_host)
  add_library(nvshmem::nvshmem_host SHARED IMPORTED GLOBAL)
  set_target_properties(nvshmem::nvshmem_host PROPERTIES
    IMPORTED_LOCATION "${NVSHMEM_ROOT}/lib/libnvshmem_host.so.3"
    IMPORTED_SONAME "libnvshmem_host.so.3"
    INTERFACE_INCLUDE_DIRECTORIES "${NVSHMEM_ROOT}/include")
  add_library(nvshmem::nvshmem_device STATIC IMPORTED GLOBAL)
  set_target_properties(nvshmem::nvshmem_device PROPERTIES
    IMPORTED_LOCATION "${NVSHMEM_ROOT}/lib/libnvshmem_device.a"
    INTERFACE_INCLUDE_DIRECTORIES "${NVSHMEM_ROOT}/include")
  add_library(nvshmem::nvshmem INTERFACE IMPORTED GLOBAL)
  target_include_directories(nvshmem::nvshmem INTERFACE "${NVSHMEM_ROOT}/include")
  target_link_libraries(nvshmem::nvshmem INTERFACE nvshmem::nvshmem_host nvshmem::nvshmem_device
                        CUDA::cudart CUDA::cuda_driver)
  add_library(nvshmem::nvshmem_bootstrap_uid SHARED IMPORTED GLOBAL)
  set_target_properties(nvshmem::nvshmem_bootstrap_uid PROPERTIES
    IMPORTED_LOCATION "${NVSHMEM_ROOT}/lib/nvshmem_bootstrap_uid.so.3"
    IMPORTED_SONAME "nvshmem_bootstrap_uid.so.3")
endif()
set(NVSHMEM_INCLUDE_DIR "${NVSHMEM_ROOT}/include")
set(NVSHMEM_FOUND TRUE)
