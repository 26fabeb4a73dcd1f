#include "env.h"

#include <algorithm>
#include <cstdlib>

namespace hvd {

bool EnvIsSet(const char* name) {
  const char* v = std::getenv(name);
  return v != nullptr && *v != '\0';
}

std::string EnvString(const char* name, const std::string& dflt) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::string(v) : dflt;
}

int64_t EnvInt(const char* name, int64_t dflt) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return dflt;
  char* end = nullptr;
  long long r = std::strtoll(v, &end, 10);
  return end == v ? dflt : static_cast<int64_t>(r);
}

double EnvDouble(const char* name, double dflt) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return dflt;
  char* end = nullptr;
  double r = std::strtod(v, &end);
  return end == v ? dflt : r;
}

bool EnvBool(const char* name, bool dflt) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return dflt;
  std::string s(v);
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  if (s == "1" || s == "true" || s == "yes" || s == "on") return true;
  if (s == "0" || s == "false" || s == "no" || s == "off") return false;
  char* end = nullptr;
  long r = std::strtol(v, &end, 10);
  return end == v ? dflt : r > 0;
}

}  // namespace hvd
