/*
 * TEST INFRASTRUCTURE ONLY.  Minimal stand-in for <glog/logging.h>, which is not installed in this image,
 * so that the reference project's header-only amd64 attention code can be compiled in place for the
 * parity checker (oracle/ref_harness.cc).  It provides the streaming macros those headers use: fatal
 * severities and failed CHECKs abort after printing; debug forms compile to nothing (the reference
 * builds with -DNDEBUG); every other severity is discarded.
 */
#pragma once

#include <cstdlib>
#include <iostream>
#include <sstream>

namespace gh_glog_shim {

struct Sink
{
  bool fatal;
  std::ostringstream os;
  explicit Sink( bool f ) : fatal( f ) {}
  ~Sink()
  {
    if ( fatal ) {
      std::cerr << os.str() << std::endl;
      std::abort();
    }
  }
  template<typename V>
  Sink& operator<<( const V& v )
  {
    if ( fatal )
      os << v;
    return *this;
  }
  Sink& operator<<( std::ostream& ( * )( std::ostream& ) ) { return *this; }
};

struct Voidify
{
  void operator&( const Sink& ) {}
};

constexpr bool is_fatal_INFO = false;
constexpr bool is_fatal_WARNING = false;
constexpr bool is_fatal_ERROR = false;
constexpr bool is_fatal_FATAL = true;

} // namespace gh_glog_shim

#define LOG( sev ) ::gh_glog_shim::Sink( ::gh_glog_shim::is_fatal_##sev )
#define GH_SHIM_CHECK( cond )                                                                                          \
  ( cond ) ? (void)0 : ::gh_glog_shim::Voidify() & ::gh_glog_shim::Sink( true ) << "Check failed: " #cond " "
#define GH_SHIM_NOP( cond ) true ? (void)0 : ::gh_glog_shim::Voidify() & ::gh_glog_shim::Sink( false )

#define CHECK( cond ) GH_SHIM_CHECK( cond )
#define CHECK_EQ( a, b ) GH_SHIM_CHECK( ( a ) == ( b ) )
#define CHECK_NE( a, b ) GH_SHIM_CHECK( ( a ) != ( b ) )
#define CHECK_LT( a, b ) GH_SHIM_CHECK( ( a ) < ( b ) )
#define CHECK_LE( a, b ) GH_SHIM_CHECK( ( a ) <= ( b ) )
#define CHECK_GT( a, b ) GH_SHIM_CHECK( ( a ) > ( b ) )
#define CHECK_GE( a, b ) GH_SHIM_CHECK( ( a ) >= ( b ) )
#define CHECK_ERR( x ) GH_SHIM_CHECK( ( x ) != -1 )

#define DLOG( sev ) GH_SHIM_NOP( true )
#define DCHECK( cond ) GH_SHIM_NOP( cond )
#define DCHECK_EQ( a, b ) GH_SHIM_NOP( true )
#define DCHECK_NE( a, b ) GH_SHIM_NOP( true )
#define DCHECK_LT( a, b ) GH_SHIM_NOP( true )
#define DCHECK_LE( a, b ) GH_SHIM_NOP( true )
#define DCHECK_GT( a, b ) GH_SHIM_NOP( true )
#define DCHECK_GE( a, b ) GH_SHIM_NOP( true )
