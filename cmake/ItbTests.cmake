# Native test suites, registered with ctest.
#
#   itb_add_test_suite(<name> SOURCES <files...> [TORCH] [LIBS <targets...>])
#
# builds <name>_cpu from the sources and registers the ctest test <name>_cpu (label "cpu"), which runs
# `<name>_cpu --device cpu`.  With TORCH the suite is built on libtorch and the C++ frontend headers,
# and, when ITB_WITH_CUDA is on, a second binary <name>_cuda is built with -DITB_WITH_CUDA against the
# sm_100a kernels of _C.so and registered as <name>_cuda (label "cuda"), which runs
# `<name>_cuda --device cuda`.  Exit code 77 (no visible GPU) shows up as "skipped".
#
# This is the counterpart of the reference's infini_train_add_test_suite (cmake/test_macros.cmake:
# 50-156: one binary per device, CPU cases discovered, CUDA cases registered per binary, labels
# cpu / cuda, 10 s default time-out).
#
#   itb_add_compile_fail_test(<name> SOURCE <file> [INCLUDES <dirs...>])
#
# registers a ctest test that passes only when <file> does NOT compile (an EXCLUDE_FROM_ALL target
# built through `cmake --build`, WILL_FAIL).

include(CMakeParseArguments)

function(itb_add_test_suite name)
  cmake_parse_arguments(ARG "TORCH" "TIMEOUT" "SOURCES;LIBS" ${ARGN})
  if(NOT ARG_TIMEOUT)
    set(ARG_TIMEOUT 120)
  endif()
  add_executable(${name}_cpu ${ARG_SOURCES})
  target_include_directories(${name}_cpu PRIVATE ${PROJECT_SOURCE_DIR}/tests/native
                                                 ${PROJECT_SOURCE_DIR}/infinitrain_b200/csrc/runtime)
  target_link_libraries(${name}_cpu PRIVATE ${ARG_LIBS} Threads::Threads)
  if(ARG_TORCH)
    target_link_libraries(${name}_cpu PRIVATE itb_frontend)
  endif()
  add_test(NAME ${name}_cpu COMMAND ${name}_cpu --device cpu)
  set_tests_properties(${name}_cpu PROPERTIES LABELS "cpu" TIMEOUT ${ARG_TIMEOUT} SKIP_RETURN_CODE 77)

  if(ARG_TORCH AND ITB_WITH_CUDA)
    add_executable(${name}_cuda ${ARG_SOURCES})
    target_include_directories(${name}_cuda PRIVATE ${PROJECT_SOURCE_DIR}/tests/native
                                                    ${PROJECT_SOURCE_DIR}/infinitrain_b200/csrc/runtime)
    target_link_libraries(${name}_cuda PRIVATE ${ARG_LIBS} itb_frontend_cuda Threads::Threads)
    add_test(NAME ${name}_cuda COMMAND ${name}_cuda --device cuda)
    set_tests_properties(${name}_cuda PROPERTIES LABELS "cuda" TIMEOUT ${ARG_TIMEOUT} SKIP_RETURN_CODE 77)
  endif()
endfunction()

function(itb_add_compile_fail_test name)
  cmake_parse_arguments(ARG "" "SOURCE" "INCLUDES" ${ARGN})
  add_executable(${name} EXCLUDE_FROM_ALL ${ARG_SOURCE})
  target_include_directories(${name} PRIVATE ${ARG_INCLUDES})
  add_test(NAME ${name}
           COMMAND ${CMAKE_COMMAND} --build ${CMAKE_BINARY_DIR} --target ${name})
  set_tests_properties(${name} PROPERTIES WILL_FAIL TRUE LABELS "cpu" TIMEOUT 300)
endfunction()
