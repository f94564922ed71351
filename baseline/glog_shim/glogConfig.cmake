# find_package(glog) lands here (-Dglog_DIR=<this folder>): glog::glog is the header-only stand-in beside this file.
if(NOT TARGET glog::glog)
  add_library(glog::glog INTERFACE IMPORTED)
  set_target_properties(glog::glog PROPERTIES INTERFACE_INCLUDE_DIRECTORIES "${CMAKE_CURRENT_LIST_DIR}")
endif()
set(glog_FOUND TRUE)
