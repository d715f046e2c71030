* c1355 (c1355: c499 with the XORs expanded into NANDs): 558 gates, 2604 transistors
VDD vdd 0 DC 1.8
VIN0 nd0 0 PULSE(0 1.8 5e-10 20p 20p 1e-09 2e-09)
VIN1 nd1 0 PULSE(0 1.8 1e-09 20p 20p 2e-09 4e-09)
VIN2 nd2 0 PULSE(0 1.8 2e-09 20p 20p 4e-09 8e-09)
VIN3 nd3 0 PULSE(0 1.8 4e-09 20p 20p 8e-09 1.6e-08)
VIN4 nd4 0 PULSE(0 1.8 8e-09 20p 20p 1.6e-08 3.2e-08)
VIN5 nd5 0 PULSE(0 1.8 1.6e-08 20p 20p 3.2e-08 6.4e-08)
VIN6 nd6 0 PULSE(0 1.8 3.2e-08 20p 20p 6.4e-08 1.28e-07)
VIN7 nd7 0 PULSE(0 1.8 6.4e-08 20p 20p 1.28e-07 2.56e-07)
VIN8 nd8 0 PULSE(0 1.8 1.28e-07 20p 20p 2.56e-07 5.12e-07)
VIN9 nd9 0 PULSE(0 1.8 2.56e-07 20p 20p 5.12e-07 1.024e-06)
VIN10 nd10 0 PULSE(0 1.8 5.12e-07 20p 20p 1.024e-06 2.048e-06)
VIN11 nd11 0 PULSE(0 1.8 1.024e-06 20p 20p 2.048e-06 4.096e-06)
VIN12 nd12 0 PULSE(0 1.8 2.048e-06 20p 20p 4.096e-06 8.192e-06)
VIN13 nd13 0 PULSE(0 1.8 4.096e-06 20p 20p 8.192e-06 1.6384e-05)
VIN14 nd14 0 PULSE(0 1.8 8.192e-06 20p 20p 1.6384e-05 3.2768e-05)
VIN15 nd15 0 PULSE(0 1.8 1.6384e-05 20p 20p 3.2768e-05 6.5536e-05)
VIN16 nd16 0 PULSE(0 1.8 3.2768e-05 20p 20p 6.5536e-05 0.000131072)
VIN17 nd17 0 PULSE(0 1.8 6.5536e-05 20p 20p 0.000131072 0.000262144)
VIN18 nd18 0 PULSE(0 1.8 0.000131072 20p 20p 0.000262144 0.000524288)
VIN19 nd19 0 PULSE(0 1.8 0.000262144 20p 20p 0.000524288 0.001048576)
VIN20 nd20 0 PULSE(0 1.8 0.000524288 20p 20p 0.001048576 0.002097152)
VIN21 nd21 0 PULSE(0 1.8 0.001048576 20p 20p 0.002097152 0.004194304)
VIN22 nd22 0 PULSE(0 1.8 0.002097152 20p 20p 0.004194304 0.008388608)
VIN23 nd23 0 PULSE(0 1.8 0.004194304 20p 20p 0.008388608 0.016777216)
VIN24 nd24 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN25 nd25 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN26 nd26 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN27 nd27 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN28 nd28 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN29 nd29 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN30 nd30 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN31 nd31 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN32 nr0 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN33 nr1 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN34 nr2 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN35 nr3 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN36 nr4 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN37 nr5 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
VIN38 nen 0 PULSE(0 1.8 0.008388608 20p 20p 0.016777216 0.033554432)
M1 nw1 nd0 vdd vdd pch w=2u l=180n
M2 nw1 nd1 vdd vdd pch w=2u l=180n
CT1 t1 0 0.1f
M3 nw1 nd0 t1 0 nch w=1u l=180n
M4 t1 nd1 0 0 nch w=1u l=180n
Cnw1 nw1 0 2f
M5 nw2 nd0 vdd vdd pch w=2u l=180n
M6 nw2 nw1 vdd vdd pch w=2u l=180n
CT2 t2 0 0.1f
M7 nw2 nd0 t2 0 nch w=1u l=180n
M8 t2 nw1 0 0 nch w=1u l=180n
Cnw2 nw2 0 2f
M9 nw3 nd1 vdd vdd pch w=2u l=180n
M10 nw3 nw1 vdd vdd pch w=2u l=180n
CT3 t3 0 0.1f
M11 nw3 nd1 t3 0 nch w=1u l=180n
M12 t3 nw1 0 0 nch w=1u l=180n
Cnw3 nw3 0 2f
M13 nw4 nw2 vdd vdd pch w=2u l=180n
M14 nw4 nw3 vdd vdd pch w=2u l=180n
CT4 t4 0 0.1f
M15 nw4 nw2 t4 0 nch w=1u l=180n
M16 t4 nw3 0 0 nch w=1u l=180n
Cnw4 nw4 0 2f
M17 nw5 nw4 vdd vdd pch w=2u l=180n
M18 nw5 nd3 vdd vdd pch w=2u l=180n
CT5 t5 0 0.1f
M19 nw5 nw4 t5 0 nch w=1u l=180n
M20 t5 nd3 0 0 nch w=1u l=180n
Cnw5 nw5 0 2f
M21 nw6 nw4 vdd vdd pch w=2u l=180n
M22 nw6 nw5 vdd vdd pch w=2u l=180n
CT6 t6 0 0.1f
M23 nw6 nw4 t6 0 nch w=1u l=180n
M24 t6 nw5 0 0 nch w=1u l=180n
Cnw6 nw6 0 2f
M25 nw7 nd3 vdd vdd pch w=2u l=180n
M26 nw7 nw5 vdd vdd pch w=2u l=180n
CT7 t7 0 0.1f
M27 nw7 nd3 t7 0 nch w=1u l=180n
M28 t7 nw5 0 0 nch w=1u l=180n
Cnw7 nw7 0 2f
M29 nw8 nw6 vdd vdd pch w=2u l=180n
M30 nw8 nw7 vdd vdd pch w=2u l=180n
CT8 t8 0 0.1f
M31 nw8 nw6 t8 0 nch w=1u l=180n
M32 t8 nw7 0 0 nch w=1u l=180n
Cnw8 nw8 0 2f
M33 nw9 nw8 vdd vdd pch w=2u l=180n
M34 nw9 nd4 vdd vdd pch w=2u l=180n
CT9 t9 0 0.1f
M35 nw9 nw8 t9 0 nch w=1u l=180n
M36 t9 nd4 0 0 nch w=1u l=180n
Cnw9 nw9 0 2f
M37 nw10 nw8 vdd vdd pch w=2u l=180n
M38 nw10 nw9 vdd vdd pch w=2u l=180n
CT10 t10 0 0.1f
M39 nw10 nw8 t10 0 nch w=1u l=180n
M40 t10 nw9 0 0 nch w=1u l=180n
Cnw10 nw10 0 2f
M41 nw11 nd4 vdd vdd pch w=2u l=180n
M42 nw11 nw9 vdd vdd pch w=2u l=180n
CT11 t11 0 0.1f
M43 nw11 nd4 t11 0 nch w=1u l=180n
M44 t11 nw9 0 0 nch w=1u l=180n
Cnw11 nw11 0 2f
M45 nw12 nw10 vdd vdd pch w=2u l=180n
M46 nw12 nw11 vdd vdd pch w=2u l=180n
CT12 t12 0 0.1f
M47 nw12 nw10 t12 0 nch w=1u l=180n
M48 t12 nw11 0 0 nch w=1u l=180n
Cnw12 nw12 0 2f
M49 nw13 nw12 vdd vdd pch w=2u l=180n
M50 nw13 nd6 vdd vdd pch w=2u l=180n
CT13 t13 0 0.1f
M51 nw13 nw12 t13 0 nch w=1u l=180n
M52 t13 nd6 0 0 nch w=1u l=180n
Cnw13 nw13 0 2f
M53 nw14 nw12 vdd vdd pch w=2u l=180n
M54 nw14 nw13 vdd vdd pch w=2u l=180n
CT14 t14 0 0.1f
M55 nw14 nw12 t14 0 nch w=1u l=180n
M56 t14 nw13 0 0 nch w=1u l=180n
Cnw14 nw14 0 2f
M57 nw15 nd6 vdd vdd pch w=2u l=180n
M58 nw15 nw13 vdd vdd pch w=2u l=180n
CT15 t15 0 0.1f
M59 nw15 nd6 t15 0 nch w=1u l=180n
M60 t15 nw13 0 0 nch w=1u l=180n
Cnw15 nw15 0 2f
M61 nw16 nw14 vdd vdd pch w=2u l=180n
M62 nw16 nw15 vdd vdd pch w=2u l=180n
CT16 t16 0 0.1f
M63 nw16 nw14 t16 0 nch w=1u l=180n
M64 t16 nw15 0 0 nch w=1u l=180n
Cnw16 nw16 0 2f
M65 nw17 nw16 vdd vdd pch w=2u l=180n
M66 nw17 nd8 vdd vdd pch w=2u l=180n
CT17 t17 0 0.1f
M67 nw17 nw16 t17 0 nch w=1u l=180n
M68 t17 nd8 0 0 nch w=1u l=180n
Cnw17 nw17 0 2f
M69 nw18 nw16 vdd vdd pch w=2u l=180n
M70 nw18 nw17 vdd vdd pch w=2u l=180n
CT18 t18 0 0.1f
M71 nw18 nw16 t18 0 nch w=1u l=180n
M72 t18 nw17 0 0 nch w=1u l=180n
Cnw18 nw18 0 2f
M73 nw19 nd8 vdd vdd pch w=2u l=180n
M74 nw19 nw17 vdd vdd pch w=2u l=180n
CT19 t19 0 0.1f
M75 nw19 nd8 t19 0 nch w=1u l=180n
M76 t19 nw17 0 0 nch w=1u l=180n
Cnw19 nw19 0 2f
M77 nw20 nw18 vdd vdd pch w=2u l=180n
M78 nw20 nw19 vdd vdd pch w=2u l=180n
CT20 t20 0 0.1f
M79 nw20 nw18 t20 0 nch w=1u l=180n
M80 t20 nw19 0 0 nch w=1u l=180n
Cnw20 nw20 0 2f
M81 nw21 nw20 vdd vdd pch w=2u l=180n
M82 nw21 nd10 vdd vdd pch w=2u l=180n
CT21 t21 0 0.1f
M83 nw21 nw20 t21 0 nch w=1u l=180n
M84 t21 nd10 0 0 nch w=1u l=180n
Cnw21 nw21 0 2f
M85 nw22 nw20 vdd vdd pch w=2u l=180n
M86 nw22 nw21 vdd vdd pch w=2u l=180n
CT22 t22 0 0.1f
M87 nw22 nw20 t22 0 nch w=1u l=180n
M88 t22 nw21 0 0 nch w=1u l=180n
Cnw22 nw22 0 2f
M89 nw23 nd10 vdd vdd pch w=2u l=180n
M90 nw23 nw21 vdd vdd pch w=2u l=180n
CT23 t23 0 0.1f
M91 nw23 nd10 t23 0 nch w=1u l=180n
M92 t23 nw21 0 0 nch w=1u l=180n
Cnw23 nw23 0 2f
M93 nw24 nw22 vdd vdd pch w=2u l=180n
M94 nw24 nw23 vdd vdd pch w=2u l=180n
CT24 t24 0 0.1f
M95 nw24 nw22 t24 0 nch w=1u l=180n
M96 t24 nw23 0 0 nch w=1u l=180n
Cnw24 nw24 0 2f
M97 nw25 nw24 vdd vdd pch w=2u l=180n
M98 nw25 nd11 vdd vdd pch w=2u l=180n
CT25 t25 0 0.1f
M99 nw25 nw24 t25 0 nch w=1u l=180n
M100 t25 nd11 0 0 nch w=1u l=180n
Cnw25 nw25 0 2f
M101 nw26 nw24 vdd vdd pch w=2u l=180n
M102 nw26 nw25 vdd vdd pch w=2u l=180n
CT26 t26 0 0.1f
M103 nw26 nw24 t26 0 nch w=1u l=180n
M104 t26 nw25 0 0 nch w=1u l=180n
Cnw26 nw26 0 2f
M105 nw27 nd11 vdd vdd pch w=2u l=180n
M106 nw27 nw25 vdd vdd pch w=2u l=180n
CT27 t27 0 0.1f
M107 nw27 nd11 t27 0 nch w=1u l=180n
M108 t27 nw25 0 0 nch w=1u l=180n
Cnw27 nw27 0 2f
M109 nw28 nw26 vdd vdd pch w=2u l=180n
M110 nw28 nw27 vdd vdd pch w=2u l=180n
CT28 t28 0 0.1f
M111 nw28 nw26 t28 0 nch w=1u l=180n
M112 t28 nw27 0 0 nch w=1u l=180n
Cnw28 nw28 0 2f
M113 nw29 nw28 vdd vdd pch w=2u l=180n
M114 nw29 nd13 vdd vdd pch w=2u l=180n
CT29 t29 0 0.1f
M115 nw29 nw28 t29 0 nch w=1u l=180n
M116 t29 nd13 0 0 nch w=1u l=180n
Cnw29 nw29 0 2f
M117 nw30 nw28 vdd vdd pch w=2u l=180n
M118 nw30 nw29 vdd vdd pch w=2u l=180n
CT30 t30 0 0.1f
M119 nw30 nw28 t30 0 nch w=1u l=180n
M120 t30 nw29 0 0 nch w=1u l=180n
Cnw30 nw30 0 2f
M121 nw31 nd13 vdd vdd pch w=2u l=180n
M122 nw31 nw29 vdd vdd pch w=2u l=180n
CT31 t31 0 0.1f
M123 nw31 nd13 t31 0 nch w=1u l=180n
M124 t31 nw29 0 0 nch w=1u l=180n
Cnw31 nw31 0 2f
M125 nw32 nw30 vdd vdd pch w=2u l=180n
M126 nw32 nw31 vdd vdd pch w=2u l=180n
CT32 t32 0 0.1f
M127 nw32 nw30 t32 0 nch w=1u l=180n
M128 t32 nw31 0 0 nch w=1u l=180n
Cnw32 nw32 0 2f
M129 nw33 nw32 vdd vdd pch w=2u l=180n
M130 nw33 nd15 vdd vdd pch w=2u l=180n
CT33 t33 0 0.1f
M131 nw33 nw32 t33 0 nch w=1u l=180n
M132 t33 nd15 0 0 nch w=1u l=180n
Cnw33 nw33 0 2f
M133 nw34 nw32 vdd vdd pch w=2u l=180n
M134 nw34 nw33 vdd vdd pch w=2u l=180n
CT34 t34 0 0.1f
M135 nw34 nw32 t34 0 nch w=1u l=180n
M136 t34 nw33 0 0 nch w=1u l=180n
Cnw34 nw34 0 2f
M137 nw35 nd15 vdd vdd pch w=2u l=180n
M138 nw35 nw33 vdd vdd pch w=2u l=180n
CT35 t35 0 0.1f
M139 nw35 nd15 t35 0 nch w=1u l=180n
M140 t35 nw33 0 0 nch w=1u l=180n
Cnw35 nw35 0 2f
M141 nw36 nw34 vdd vdd pch w=2u l=180n
M142 nw36 nw35 vdd vdd pch w=2u l=180n
CT36 t36 0 0.1f
M143 nw36 nw34 t36 0 nch w=1u l=180n
M144 t36 nw35 0 0 nch w=1u l=180n
Cnw36 nw36 0 2f
M145 nw37 nw36 vdd vdd pch w=2u l=180n
M146 nw37 nd17 vdd vdd pch w=2u l=180n
CT37 t37 0 0.1f
M147 nw37 nw36 t37 0 nch w=1u l=180n
M148 t37 nd17 0 0 nch w=1u l=180n
Cnw37 nw37 0 2f
M149 nw38 nw36 vdd vdd pch w=2u l=180n
M150 nw38 nw37 vdd vdd pch w=2u l=180n
CT38 t38 0 0.1f
M151 nw38 nw36 t38 0 nch w=1u l=180n
M152 t38 nw37 0 0 nch w=1u l=180n
Cnw38 nw38 0 2f
M153 nw39 nd17 vdd vdd pch w=2u l=180n
M154 nw39 nw37 vdd vdd pch w=2u l=180n
CT39 t39 0 0.1f
M155 nw39 nd17 t39 0 nch w=1u l=180n
M156 t39 nw37 0 0 nch w=1u l=180n
Cnw39 nw39 0 2f
M157 nw40 nw38 vdd vdd pch w=2u l=180n
M158 nw40 nw39 vdd vdd pch w=2u l=180n
CT40 t40 0 0.1f
M159 nw40 nw38 t40 0 nch w=1u l=180n
M160 t40 nw39 0 0 nch w=1u l=180n
Cnw40 nw40 0 2f
M161 nw41 nw40 vdd vdd pch w=2u l=180n
M162 nw41 nd19 vdd vdd pch w=2u l=180n
CT41 t41 0 0.1f
M163 nw41 nw40 t41 0 nch w=1u l=180n
M164 t41 nd19 0 0 nch w=1u l=180n
Cnw41 nw41 0 2f
M165 nw42 nw40 vdd vdd pch w=2u l=180n
M166 nw42 nw41 vdd vdd pch w=2u l=180n
CT42 t42 0 0.1f
M167 nw42 nw40 t42 0 nch w=1u l=180n
M168 t42 nw41 0 0 nch w=1u l=180n
Cnw42 nw42 0 2f
M169 nw43 nd19 vdd vdd pch w=2u l=180n
M170 nw43 nw41 vdd vdd pch w=2u l=180n
CT43 t43 0 0.1f
M171 nw43 nd19 t43 0 nch w=1u l=180n
M172 t43 nw41 0 0 nch w=1u l=180n
Cnw43 nw43 0 2f
M173 nw44 nw42 vdd vdd pch w=2u l=180n
M174 nw44 nw43 vdd vdd pch w=2u l=180n
CT44 t44 0 0.1f
M175 nw44 nw42 t44 0 nch w=1u l=180n
M176 t44 nw43 0 0 nch w=1u l=180n
Cnw44 nw44 0 2f
M177 nw45 nw44 vdd vdd pch w=2u l=180n
M178 nw45 nd21 vdd vdd pch w=2u l=180n
CT45 t45 0 0.1f
M179 nw45 nw44 t45 0 nch w=1u l=180n
M180 t45 nd21 0 0 nch w=1u l=180n
Cnw45 nw45 0 2f
M181 nw46 nw44 vdd vdd pch w=2u l=180n
M182 nw46 nw45 vdd vdd pch w=2u l=180n
CT46 t46 0 0.1f
M183 nw46 nw44 t46 0 nch w=1u l=180n
M184 t46 nw45 0 0 nch w=1u l=180n
Cnw46 nw46 0 2f
M185 nw47 nd21 vdd vdd pch w=2u l=180n
M186 nw47 nw45 vdd vdd pch w=2u l=180n
CT47 t47 0 0.1f
M187 nw47 nd21 t47 0 nch w=1u l=180n
M188 t47 nw45 0 0 nch w=1u l=180n
Cnw47 nw47 0 2f
M189 nw48 nw46 vdd vdd pch w=2u l=180n
M190 nw48 nw47 vdd vdd pch w=2u l=180n
CT48 t48 0 0.1f
M191 nw48 nw46 t48 0 nch w=1u l=180n
M192 t48 nw47 0 0 nch w=1u l=180n
Cnw48 nw48 0 2f
M193 nw49 nw48 vdd vdd pch w=2u l=180n
M194 nw49 nd23 vdd vdd pch w=2u l=180n
CT49 t49 0 0.1f
M195 nw49 nw48 t49 0 nch w=1u l=180n
M196 t49 nd23 0 0 nch w=1u l=180n
Cnw49 nw49 0 2f
M197 nw50 nw48 vdd vdd pch w=2u l=180n
M198 nw50 nw49 vdd vdd pch w=2u l=180n
CT50 t50 0 0.1f
M199 nw50 nw48 t50 0 nch w=1u l=180n
M200 t50 nw49 0 0 nch w=1u l=180n
Cnw50 nw50 0 2f
M201 nw51 nd23 vdd vdd pch w=2u l=180n
M202 nw51 nw49 vdd vdd pch w=2u l=180n
CT51 t51 0 0.1f
M203 nw51 nd23 t51 0 nch w=1u l=180n
M204 t51 nw49 0 0 nch w=1u l=180n
Cnw51 nw51 0 2f
M205 nw52 nw50 vdd vdd pch w=2u l=180n
M206 nw52 nw51 vdd vdd pch w=2u l=180n
CT52 t52 0 0.1f
M207 nw52 nw50 t52 0 nch w=1u l=180n
M208 t52 nw51 0 0 nch w=1u l=180n
Cnw52 nw52 0 2f
M209 nw53 nw52 vdd vdd pch w=2u l=180n
M210 nw53 nd25 vdd vdd pch w=2u l=180n
CT53 t53 0 0.1f
M211 nw53 nw52 t53 0 nch w=1u l=180n
M212 t53 nd25 0 0 nch w=1u l=180n
Cnw53 nw53 0 2f
M213 nw54 nw52 vdd vdd pch w=2u l=180n
M214 nw54 nw53 vdd vdd pch w=2u l=180n
CT54 t54 0 0.1f
M215 nw54 nw52 t54 0 nch w=1u l=180n
M216 t54 nw53 0 0 nch w=1u l=180n
Cnw54 nw54 0 2f
M217 nw55 nd25 vdd vdd pch w=2u l=180n
M218 nw55 nw53 vdd vdd pch w=2u l=180n
CT55 t55 0 0.1f
M219 nw55 nd25 t55 0 nch w=1u l=180n
M220 t55 nw53 0 0 nch w=1u l=180n
Cnw55 nw55 0 2f
M221 nw56 nw54 vdd vdd pch w=2u l=180n
M222 nw56 nw55 vdd vdd pch w=2u l=180n
CT56 t56 0 0.1f
M223 nw56 nw54 t56 0 nch w=1u l=180n
M224 t56 nw55 0 0 nch w=1u l=180n
Cnw56 nw56 0 2f
M225 nw57 nw56 vdd vdd pch w=2u l=180n
M226 nw57 nd26 vdd vdd pch w=2u l=180n
CT57 t57 0 0.1f
M227 nw57 nw56 t57 0 nch w=1u l=180n
M228 t57 nd26 0 0 nch w=1u l=180n
Cnw57 nw57 0 2f
M229 nw58 nw56 vdd vdd pch w=2u l=180n
M230 nw58 nw57 vdd vdd pch w=2u l=180n
CT58 t58 0 0.1f
M231 nw58 nw56 t58 0 nch w=1u l=180n
M232 t58 nw57 0 0 nch w=1u l=180n
Cnw58 nw58 0 2f
M233 nw59 nd26 vdd vdd pch w=2u l=180n
M234 nw59 nw57 vdd vdd pch w=2u l=180n
CT59 t59 0 0.1f
M235 nw59 nd26 t59 0 nch w=1u l=180n
M236 t59 nw57 0 0 nch w=1u l=180n
Cnw59 nw59 0 2f
M237 nw60 nw58 vdd vdd pch w=2u l=180n
M238 nw60 nw59 vdd vdd pch w=2u l=180n
CT60 t60 0 0.1f
M239 nw60 nw58 t60 0 nch w=1u l=180n
M240 t60 nw59 0 0 nch w=1u l=180n
Cnw60 nw60 0 2f
M241 nw61 nw60 vdd vdd pch w=2u l=180n
M242 nw61 nd28 vdd vdd pch w=2u l=180n
CT61 t61 0 0.1f
M243 nw61 nw60 t61 0 nch w=1u l=180n
M244 t61 nd28 0 0 nch w=1u l=180n
Cnw61 nw61 0 2f
M245 nw62 nw60 vdd vdd pch w=2u l=180n
M246 nw62 nw61 vdd vdd pch w=2u l=180n
CT62 t62 0 0.1f
M247 nw62 nw60 t62 0 nch w=1u l=180n
M248 t62 nw61 0 0 nch w=1u l=180n
Cnw62 nw62 0 2f
M249 nw63 nd28 vdd vdd pch w=2u l=180n
M250 nw63 nw61 vdd vdd pch w=2u l=180n
CT63 t63 0 0.1f
M251 nw63 nd28 t63 0 nch w=1u l=180n
M252 t63 nw61 0 0 nch w=1u l=180n
Cnw63 nw63 0 2f
M253 nw64 nw62 vdd vdd pch w=2u l=180n
M254 nw64 nw63 vdd vdd pch w=2u l=180n
CT64 t64 0 0.1f
M255 nw64 nw62 t64 0 nch w=1u l=180n
M256 t64 nw63 0 0 nch w=1u l=180n
Cnw64 nw64 0 2f
M257 nw65 nw64 vdd vdd pch w=2u l=180n
M258 nw65 nd30 vdd vdd pch w=2u l=180n
CT65 t65 0 0.1f
M259 nw65 nw64 t65 0 nch w=1u l=180n
M260 t65 nd30 0 0 nch w=1u l=180n
Cnw65 nw65 0 2f
M261 nw66 nw64 vdd vdd pch w=2u l=180n
M262 nw66 nw65 vdd vdd pch w=2u l=180n
CT66 t66 0 0.1f
M263 nw66 nw64 t66 0 nch w=1u l=180n
M264 t66 nw65 0 0 nch w=1u l=180n
Cnw66 nw66 0 2f
M265 nw67 nd30 vdd vdd pch w=2u l=180n
M266 nw67 nw65 vdd vdd pch w=2u l=180n
CT67 t67 0 0.1f
M267 nw67 nd30 t67 0 nch w=1u l=180n
M268 t67 nw65 0 0 nch w=1u l=180n
Cnw67 nw67 0 2f
M269 nw68 nw66 vdd vdd pch w=2u l=180n
M270 nw68 nw67 vdd vdd pch w=2u l=180n
CT68 t68 0 0.1f
M271 nw68 nw66 t68 0 nch w=1u l=180n
M272 t68 nw67 0 0 nch w=1u l=180n
Cnw68 nw68 0 2f
M273 nw69 nw68 vdd vdd pch w=2u l=180n
M274 nw69 nr0 vdd vdd pch w=2u l=180n
CT69 t69 0 0.1f
M275 nw69 nw68 t69 0 nch w=1u l=180n
M276 t69 nr0 0 0 nch w=1u l=180n
Cnw69 nw69 0 2f
M277 nw70 nw68 vdd vdd pch w=2u l=180n
M278 nw70 nw69 vdd vdd pch w=2u l=180n
CT70 t70 0 0.1f
M279 nw70 nw68 t70 0 nch w=1u l=180n
M280 t70 nw69 0 0 nch w=1u l=180n
Cnw70 nw70 0 2f
M281 nw71 nr0 vdd vdd pch w=2u l=180n
M282 nw71 nw69 vdd vdd pch w=2u l=180n
CT71 t71 0 0.1f
M283 nw71 nr0 t71 0 nch w=1u l=180n
M284 t71 nw69 0 0 nch w=1u l=180n
Cnw71 nw71 0 2f
M285 nw72 nw70 vdd vdd pch w=2u l=180n
M286 nw72 nw71 vdd vdd pch w=2u l=180n
CT72 t72 0 0.1f
M287 nw72 nw70 t72 0 nch w=1u l=180n
M288 t72 nw71 0 0 nch w=1u l=180n
Cnw72 nw72 0 2f
M289 nw73 nd0 vdd vdd pch w=2u l=180n
M290 nw73 nd2 vdd vdd pch w=2u l=180n
CT73 t73 0 0.1f
M291 nw73 nd0 t73 0 nch w=1u l=180n
M292 t73 nd2 0 0 nch w=1u l=180n
Cnw73 nw73 0 2f
M293 nw74 nd0 vdd vdd pch w=2u l=180n
M294 nw74 nw73 vdd vdd pch w=2u l=180n
CT74 t74 0 0.1f
M295 nw74 nd0 t74 0 nch w=1u l=180n
M296 t74 nw73 0 0 nch w=1u l=180n
Cnw74 nw74 0 2f
M297 nw75 nd2 vdd vdd pch w=2u l=180n
M298 nw75 nw73 vdd vdd pch w=2u l=180n
CT75 t75 0 0.1f
M299 nw75 nd2 t75 0 nch w=1u l=180n
M300 t75 nw73 0 0 nch w=1u l=180n
Cnw75 nw75 0 2f
M301 nw76 nw74 vdd vdd pch w=2u l=180n
M302 nw76 nw75 vdd vdd pch w=2u l=180n
CT76 t76 0 0.1f
M303 nw76 nw74 t76 0 nch w=1u l=180n
M304 t76 nw75 0 0 nch w=1u l=180n
Cnw76 nw76 0 2f
M305 nw77 nw76 vdd vdd pch w=2u l=180n
M306 nw77 nd3 vdd vdd pch w=2u l=180n
CT77 t77 0 0.1f
M307 nw77 nw76 t77 0 nch w=1u l=180n
M308 t77 nd3 0 0 nch w=1u l=180n
Cnw77 nw77 0 2f
M309 nw78 nw76 vdd vdd pch w=2u l=180n
M310 nw78 nw77 vdd vdd pch w=2u l=180n
CT78 t78 0 0.1f
M311 nw78 nw76 t78 0 nch w=1u l=180n
M312 t78 nw77 0 0 nch w=1u l=180n
Cnw78 nw78 0 2f
M313 nw79 nd3 vdd vdd pch w=2u l=180n
M314 nw79 nw77 vdd vdd pch w=2u l=180n
CT79 t79 0 0.1f
M315 nw79 nd3 t79 0 nch w=1u l=180n
M316 t79 nw77 0 0 nch w=1u l=180n
Cnw79 nw79 0 2f
M317 nw80 nw78 vdd vdd pch w=2u l=180n
M318 nw80 nw79 vdd vdd pch w=2u l=180n
CT80 t80 0 0.1f
M319 nw80 nw78 t80 0 nch w=1u l=180n
M320 t80 nw79 0 0 nch w=1u l=180n
Cnw80 nw80 0 2f
M321 nw81 nw80 vdd vdd pch w=2u l=180n
M322 nw81 nd5 vdd vdd pch w=2u l=180n
CT81 t81 0 0.1f
M323 nw81 nw80 t81 0 nch w=1u l=180n
M324 t81 nd5 0 0 nch w=1u l=180n
Cnw81 nw81 0 2f
M325 nw82 nw80 vdd vdd pch w=2u l=180n
M326 nw82 nw81 vdd vdd pch w=2u l=180n
CT82 t82 0 0.1f
M327 nw82 nw80 t82 0 nch w=1u l=180n
M328 t82 nw81 0 0 nch w=1u l=180n
Cnw82 nw82 0 2f
M329 nw83 nd5 vdd vdd pch w=2u l=180n
M330 nw83 nw81 vdd vdd pch w=2u l=180n
CT83 t83 0 0.1f
M331 nw83 nd5 t83 0 nch w=1u l=180n
M332 t83 nw81 0 0 nch w=1u l=180n
Cnw83 nw83 0 2f
M333 nw84 nw82 vdd vdd pch w=2u l=180n
M334 nw84 nw83 vdd vdd pch w=2u l=180n
CT84 t84 0 0.1f
M335 nw84 nw82 t84 0 nch w=1u l=180n
M336 t84 nw83 0 0 nch w=1u l=180n
Cnw84 nw84 0 2f
M337 nw85 nw84 vdd vdd pch w=2u l=180n
M338 nw85 nd6 vdd vdd pch w=2u l=180n
CT85 t85 0 0.1f
M339 nw85 nw84 t85 0 nch w=1u l=180n
M340 t85 nd6 0 0 nch w=1u l=180n
Cnw85 nw85 0 2f
M341 nw86 nw84 vdd vdd pch w=2u l=180n
M342 nw86 nw85 vdd vdd pch w=2u l=180n
CT86 t86 0 0.1f
M343 nw86 nw84 t86 0 nch w=1u l=180n
M344 t86 nw85 0 0 nch w=1u l=180n
Cnw86 nw86 0 2f
M345 nw87 nd6 vdd vdd pch w=2u l=180n
M346 nw87 nw85 vdd vdd pch w=2u l=180n
CT87 t87 0 0.1f
M347 nw87 nd6 t87 0 nch w=1u l=180n
M348 t87 nw85 0 0 nch w=1u l=180n
Cnw87 nw87 0 2f
M349 nw88 nw86 vdd vdd pch w=2u l=180n
M350 nw88 nw87 vdd vdd pch w=2u l=180n
CT88 t88 0 0.1f
M351 nw88 nw86 t88 0 nch w=1u l=180n
M352 t88 nw87 0 0 nch w=1u l=180n
Cnw88 nw88 0 2f
M353 nw89 nw88 vdd vdd pch w=2u l=180n
M354 nw89 nd9 vdd vdd pch w=2u l=180n
CT89 t89 0 0.1f
M355 nw89 nw88 t89 0 nch w=1u l=180n
M356 t89 nd9 0 0 nch w=1u l=180n
Cnw89 nw89 0 2f
M357 nw90 nw88 vdd vdd pch w=2u l=180n
M358 nw90 nw89 vdd vdd pch w=2u l=180n
CT90 t90 0 0.1f
M359 nw90 nw88 t90 0 nch w=1u l=180n
M360 t90 nw89 0 0 nch w=1u l=180n
Cnw90 nw90 0 2f
M361 nw91 nd9 vdd vdd pch w=2u l=180n
M362 nw91 nw89 vdd vdd pch w=2u l=180n
CT91 t91 0 0.1f
M363 nw91 nd9 t91 0 nch w=1u l=180n
M364 t91 nw89 0 0 nch w=1u l=180n
Cnw91 nw91 0 2f
M365 nw92 nw90 vdd vdd pch w=2u l=180n
M366 nw92 nw91 vdd vdd pch w=2u l=180n
CT92 t92 0 0.1f
M367 nw92 nw90 t92 0 nch w=1u l=180n
M368 t92 nw91 0 0 nch w=1u l=180n
Cnw92 nw92 0 2f
M369 nw93 nw92 vdd vdd pch w=2u l=180n
M370 nw93 nd10 vdd vdd pch w=2u l=180n
CT93 t93 0 0.1f
M371 nw93 nw92 t93 0 nch w=1u l=180n
M372 t93 nd10 0 0 nch w=1u l=180n
Cnw93 nw93 0 2f
M373 nw94 nw92 vdd vdd pch w=2u l=180n
M374 nw94 nw93 vdd vdd pch w=2u l=180n
CT94 t94 0 0.1f
M375 nw94 nw92 t94 0 nch w=1u l=180n
M376 t94 nw93 0 0 nch w=1u l=180n
Cnw94 nw94 0 2f
M377 nw95 nd10 vdd vdd pch w=2u l=180n
M378 nw95 nw93 vdd vdd pch w=2u l=180n
CT95 t95 0 0.1f
M379 nw95 nd10 t95 0 nch w=1u l=180n
M380 t95 nw93 0 0 nch w=1u l=180n
Cnw95 nw95 0 2f
M381 nw96 nw94 vdd vdd pch w=2u l=180n
M382 nw96 nw95 vdd vdd pch w=2u l=180n
CT96 t96 0 0.1f
M383 nw96 nw94 t96 0 nch w=1u l=180n
M384 t96 nw95 0 0 nch w=1u l=180n
Cnw96 nw96 0 2f
M385 nw97 nw96 vdd vdd pch w=2u l=180n
M386 nw97 nd12 vdd vdd pch w=2u l=180n
CT97 t97 0 0.1f
M387 nw97 nw96 t97 0 nch w=1u l=180n
M388 t97 nd12 0 0 nch w=1u l=180n
Cnw97 nw97 0 2f
M389 nw98 nw96 vdd vdd pch w=2u l=180n
M390 nw98 nw97 vdd vdd pch w=2u l=180n
CT98 t98 0 0.1f
M391 nw98 nw96 t98 0 nch w=1u l=180n
M392 t98 nw97 0 0 nch w=1u l=180n
Cnw98 nw98 0 2f
M393 nw99 nd12 vdd vdd pch w=2u l=180n
M394 nw99 nw97 vdd vdd pch w=2u l=180n
CT99 t99 0 0.1f
M395 nw99 nd12 t99 0 nch w=1u l=180n
M396 t99 nw97 0 0 nch w=1u l=180n
Cnw99 nw99 0 2f
M397 nw100 nw98 vdd vdd pch w=2u l=180n
M398 nw100 nw99 vdd vdd pch w=2u l=180n
CT100 t100 0 0.1f
M399 nw100 nw98 t100 0 nch w=1u l=180n
M400 t100 nw99 0 0 nch w=1u l=180n
Cnw100 nw100 0 2f
M401 nw101 nw100 vdd vdd pch w=2u l=180n
M402 nw101 nd13 vdd vdd pch w=2u l=180n
CT101 t101 0 0.1f
M403 nw101 nw100 t101 0 nch w=1u l=180n
M404 t101 nd13 0 0 nch w=1u l=180n
Cnw101 nw101 0 2f
M405 nw102 nw100 vdd vdd pch w=2u l=180n
M406 nw102 nw101 vdd vdd pch w=2u l=180n
CT102 t102 0 0.1f
M407 nw102 nw100 t102 0 nch w=1u l=180n
M408 t102 nw101 0 0 nch w=1u l=180n
Cnw102 nw102 0 2f
M409 nw103 nd13 vdd vdd pch w=2u l=180n
M410 nw103 nw101 vdd vdd pch w=2u l=180n
CT103 t103 0 0.1f
M411 nw103 nd13 t103 0 nch w=1u l=180n
M412 t103 nw101 0 0 nch w=1u l=180n
Cnw103 nw103 0 2f
M413 nw104 nw102 vdd vdd pch w=2u l=180n
M414 nw104 nw103 vdd vdd pch w=2u l=180n
CT104 t104 0 0.1f
M415 nw104 nw102 t104 0 nch w=1u l=180n
M416 t104 nw103 0 0 nch w=1u l=180n
Cnw104 nw104 0 2f
M417 nw105 nw104 vdd vdd pch w=2u l=180n
M418 nw105 nd16 vdd vdd pch w=2u l=180n
CT105 t105 0 0.1f
M419 nw105 nw104 t105 0 nch w=1u l=180n
M420 t105 nd16 0 0 nch w=1u l=180n
Cnw105 nw105 0 2f
M421 nw106 nw104 vdd vdd pch w=2u l=180n
M422 nw106 nw105 vdd vdd pch w=2u l=180n
CT106 t106 0 0.1f
M423 nw106 nw104 t106 0 nch w=1u l=180n
M424 t106 nw105 0 0 nch w=1u l=180n
Cnw106 nw106 0 2f
M425 nw107 nd16 vdd vdd pch w=2u l=180n
M426 nw107 nw105 vdd vdd pch w=2u l=180n
CT107 t107 0 0.1f
M427 nw107 nd16 t107 0 nch w=1u l=180n
M428 t107 nw105 0 0 nch w=1u l=180n
Cnw107 nw107 0 2f
M429 nw108 nw106 vdd vdd pch w=2u l=180n
M430 nw108 nw107 vdd vdd pch w=2u l=180n
CT108 t108 0 0.1f
M431 nw108 nw106 t108 0 nch w=1u l=180n
M432 t108 nw107 0 0 nch w=1u l=180n
Cnw108 nw108 0 2f
M433 nw109 nw108 vdd vdd pch w=2u l=180n
M434 nw109 nd17 vdd vdd pch w=2u l=180n
CT109 t109 0 0.1f
M435 nw109 nw108 t109 0 nch w=1u l=180n
M436 t109 nd17 0 0 nch w=1u l=180n
Cnw109 nw109 0 2f
M437 nw110 nw108 vdd vdd pch w=2u l=180n
M438 nw110 nw109 vdd vdd pch w=2u l=180n
CT110 t110 0 0.1f
M439 nw110 nw108 t110 0 nch w=1u l=180n
M440 t110 nw109 0 0 nch w=1u l=180n
Cnw110 nw110 0 2f
M441 nw111 nd17 vdd vdd pch w=2u l=180n
M442 nw111 nw109 vdd vdd pch w=2u l=180n
CT111 t111 0 0.1f
M443 nw111 nd17 t111 0 nch w=1u l=180n
M444 t111 nw109 0 0 nch w=1u l=180n
Cnw111 nw111 0 2f
M445 nw112 nw110 vdd vdd pch w=2u l=180n
M446 nw112 nw111 vdd vdd pch w=2u l=180n
CT112 t112 0 0.1f
M447 nw112 nw110 t112 0 nch w=1u l=180n
M448 t112 nw111 0 0 nch w=1u l=180n
Cnw112 nw112 0 2f
M449 nw113 nw112 vdd vdd pch w=2u l=180n
M450 nw113 nd20 vdd vdd pch w=2u l=180n
CT113 t113 0 0.1f
M451 nw113 nw112 t113 0 nch w=1u l=180n
M452 t113 nd20 0 0 nch w=1u l=180n
Cnw113 nw113 0 2f
M453 nw114 nw112 vdd vdd pch w=2u l=180n
M454 nw114 nw113 vdd vdd pch w=2u l=180n
CT114 t114 0 0.1f
M455 nw114 nw112 t114 0 nch w=1u l=180n
M456 t114 nw113 0 0 nch w=1u l=180n
Cnw114 nw114 0 2f
M457 nw115 nd20 vdd vdd pch w=2u l=180n
M458 nw115 nw113 vdd vdd pch w=2u l=180n
CT115 t115 0 0.1f
M459 nw115 nd20 t115 0 nch w=1u l=180n
M460 t115 nw113 0 0 nch w=1u l=180n
Cnw115 nw115 0 2f
M461 nw116 nw114 vdd vdd pch w=2u l=180n
M462 nw116 nw115 vdd vdd pch w=2u l=180n
CT116 t116 0 0.1f
M463 nw116 nw114 t116 0 nch w=1u l=180n
M464 t116 nw115 0 0 nch w=1u l=180n
Cnw116 nw116 0 2f
M465 nw117 nw116 vdd vdd pch w=2u l=180n
M466 nw117 nd21 vdd vdd pch w=2u l=180n
CT117 t117 0 0.1f
M467 nw117 nw116 t117 0 nch w=1u l=180n
M468 t117 nd21 0 0 nch w=1u l=180n
Cnw117 nw117 0 2f
M469 nw118 nw116 vdd vdd pch w=2u l=180n
M470 nw118 nw117 vdd vdd pch w=2u l=180n
CT118 t118 0 0.1f
M471 nw118 nw116 t118 0 nch w=1u l=180n
M472 t118 nw117 0 0 nch w=1u l=180n
Cnw118 nw118 0 2f
M473 nw119 nd21 vdd vdd pch w=2u l=180n
M474 nw119 nw117 vdd vdd pch w=2u l=180n
CT119 t119 0 0.1f
M475 nw119 nd21 t119 0 nch w=1u l=180n
M476 t119 nw117 0 0 nch w=1u l=180n
Cnw119 nw119 0 2f
M477 nw120 nw118 vdd vdd pch w=2u l=180n
M478 nw120 nw119 vdd vdd pch w=2u l=180n
CT120 t120 0 0.1f
M479 nw120 nw118 t120 0 nch w=1u l=180n
M480 t120 nw119 0 0 nch w=1u l=180n
Cnw120 nw120 0 2f
M481 nw121 nw120 vdd vdd pch w=2u l=180n
M482 nw121 nd24 vdd vdd pch w=2u l=180n
CT121 t121 0 0.1f
M483 nw121 nw120 t121 0 nch w=1u l=180n
M484 t121 nd24 0 0 nch w=1u l=180n
Cnw121 nw121 0 2f
M485 nw122 nw120 vdd vdd pch w=2u l=180n
M486 nw122 nw121 vdd vdd pch w=2u l=180n
CT122 t122 0 0.1f
M487 nw122 nw120 t122 0 nch w=1u l=180n
M488 t122 nw121 0 0 nch w=1u l=180n
Cnw122 nw122 0 2f
M489 nw123 nd24 vdd vdd pch w=2u l=180n
M490 nw123 nw121 vdd vdd pch w=2u l=180n
CT123 t123 0 0.1f
M491 nw123 nd24 t123 0 nch w=1u l=180n
M492 t123 nw121 0 0 nch w=1u l=180n
Cnw123 nw123 0 2f
M493 nw124 nw122 vdd vdd pch w=2u l=180n
M494 nw124 nw123 vdd vdd pch w=2u l=180n
CT124 t124 0 0.1f
M495 nw124 nw122 t124 0 nch w=1u l=180n
M496 t124 nw123 0 0 nch w=1u l=180n
Cnw124 nw124 0 2f
M497 nw125 nw124 vdd vdd pch w=2u l=180n
M498 nw125 nd25 vdd vdd pch w=2u l=180n
CT125 t125 0 0.1f
M499 nw125 nw124 t125 0 nch w=1u l=180n
M500 t125 nd25 0 0 nch w=1u l=180n
Cnw125 nw125 0 2f
M501 nw126 nw124 vdd vdd pch w=2u l=180n
M502 nw126 nw125 vdd vdd pch w=2u l=180n
CT126 t126 0 0.1f
M503 nw126 nw124 t126 0 nch w=1u l=180n
M504 t126 nw125 0 0 nch w=1u l=180n
Cnw126 nw126 0 2f
M505 nw127 nd25 vdd vdd pch w=2u l=180n
M506 nw127 nw125 vdd vdd pch w=2u l=180n
CT127 t127 0 0.1f
M507 nw127 nd25 t127 0 nch w=1u l=180n
M508 t127 nw125 0 0 nch w=1u l=180n
Cnw127 nw127 0 2f
M509 nw128 nw126 vdd vdd pch w=2u l=180n
M510 nw128 nw127 vdd vdd pch w=2u l=180n
CT128 t128 0 0.1f
M511 nw128 nw126 t128 0 nch w=1u l=180n
M512 t128 nw127 0 0 nch w=1u l=180n
Cnw128 nw128 0 2f
M513 nw129 nw128 vdd vdd pch w=2u l=180n
M514 nw129 nd27 vdd vdd pch w=2u l=180n
CT129 t129 0 0.1f
M515 nw129 nw128 t129 0 nch w=1u l=180n
M516 t129 nd27 0 0 nch w=1u l=180n
Cnw129 nw129 0 2f
M517 nw130 nw128 vdd vdd pch w=2u l=180n
M518 nw130 nw129 vdd vdd pch w=2u l=180n
CT130 t130 0 0.1f
M519 nw130 nw128 t130 0 nch w=1u l=180n
M520 t130 nw129 0 0 nch w=1u l=180n
Cnw130 nw130 0 2f
M521 nw131 nd27 vdd vdd pch w=2u l=180n
M522 nw131 nw129 vdd vdd pch w=2u l=180n
CT131 t131 0 0.1f
M523 nw131 nd27 t131 0 nch w=1u l=180n
M524 t131 nw129 0 0 nch w=1u l=180n
Cnw131 nw131 0 2f
M525 nw132 nw130 vdd vdd pch w=2u l=180n
M526 nw132 nw131 vdd vdd pch w=2u l=180n
CT132 t132 0 0.1f
M527 nw132 nw130 t132 0 nch w=1u l=180n
M528 t132 nw131 0 0 nch w=1u l=180n
Cnw132 nw132 0 2f
M529 nw133 nw132 vdd vdd pch w=2u l=180n
M530 nw133 nd28 vdd vdd pch w=2u l=180n
CT133 t133 0 0.1f
M531 nw133 nw132 t133 0 nch w=1u l=180n
M532 t133 nd28 0 0 nch w=1u l=180n
Cnw133 nw133 0 2f
M533 nw134 nw132 vdd vdd pch w=2u l=180n
M534 nw134 nw133 vdd vdd pch w=2u l=180n
CT134 t134 0 0.1f
M535 nw134 nw132 t134 0 nch w=1u l=180n
M536 t134 nw133 0 0 nch w=1u l=180n
Cnw134 nw134 0 2f
M537 nw135 nd28 vdd vdd pch w=2u l=180n
M538 nw135 nw133 vdd vdd pch w=2u l=180n
CT135 t135 0 0.1f
M539 nw135 nd28 t135 0 nch w=1u l=180n
M540 t135 nw133 0 0 nch w=1u l=180n
Cnw135 nw135 0 2f
M541 nw136 nw134 vdd vdd pch w=2u l=180n
M542 nw136 nw135 vdd vdd pch w=2u l=180n
CT136 t136 0 0.1f
M543 nw136 nw134 t136 0 nch w=1u l=180n
M544 t136 nw135 0 0 nch w=1u l=180n
Cnw136 nw136 0 2f
M545 nw137 nw136 vdd vdd pch w=2u l=180n
M546 nw137 nd31 vdd vdd pch w=2u l=180n
CT137 t137 0 0.1f
M547 nw137 nw136 t137 0 nch w=1u l=180n
M548 t137 nd31 0 0 nch w=1u l=180n
Cnw137 nw137 0 2f
M549 nw138 nw136 vdd vdd pch w=2u l=180n
M550 nw138 nw137 vdd vdd pch w=2u l=180n
CT138 t138 0 0.1f
M551 nw138 nw136 t138 0 nch w=1u l=180n
M552 t138 nw137 0 0 nch w=1u l=180n
Cnw138 nw138 0 2f
M553 nw139 nd31 vdd vdd pch w=2u l=180n
M554 nw139 nw137 vdd vdd pch w=2u l=180n
CT139 t139 0 0.1f
M555 nw139 nd31 t139 0 nch w=1u l=180n
M556 t139 nw137 0 0 nch w=1u l=180n
Cnw139 nw139 0 2f
M557 nw140 nw138 vdd vdd pch w=2u l=180n
M558 nw140 nw139 vdd vdd pch w=2u l=180n
CT140 t140 0 0.1f
M559 nw140 nw138 t140 0 nch w=1u l=180n
M560 t140 nw139 0 0 nch w=1u l=180n
Cnw140 nw140 0 2f
M561 nw141 nw140 vdd vdd pch w=2u l=180n
M562 nw141 nr1 vdd vdd pch w=2u l=180n
CT141 t141 0 0.1f
M563 nw141 nw140 t141 0 nch w=1u l=180n
M564 t141 nr1 0 0 nch w=1u l=180n
Cnw141 nw141 0 2f
M565 nw142 nw140 vdd vdd pch w=2u l=180n
M566 nw142 nw141 vdd vdd pch w=2u l=180n
CT142 t142 0 0.1f
M567 nw142 nw140 t142 0 nch w=1u l=180n
M568 t142 nw141 0 0 nch w=1u l=180n
Cnw142 nw142 0 2f
M569 nw143 nr1 vdd vdd pch w=2u l=180n
M570 nw143 nw141 vdd vdd pch w=2u l=180n
CT143 t143 0 0.1f
M571 nw143 nr1 t143 0 nch w=1u l=180n
M572 t143 nw141 0 0 nch w=1u l=180n
Cnw143 nw143 0 2f
M573 nw144 nw142 vdd vdd pch w=2u l=180n
M574 nw144 nw143 vdd vdd pch w=2u l=180n
CT144 t144 0 0.1f
M575 nw144 nw142 t144 0 nch w=1u l=180n
M576 t144 nw143 0 0 nch w=1u l=180n
Cnw144 nw144 0 2f
M577 nw145 nd1 vdd vdd pch w=2u l=180n
M578 nw145 nd2 vdd vdd pch w=2u l=180n
CT145 t145 0 0.1f
M579 nw145 nd1 t145 0 nch w=1u l=180n
M580 t145 nd2 0 0 nch w=1u l=180n
Cnw145 nw145 0 2f
M581 nw146 nd1 vdd vdd pch w=2u l=180n
M582 nw146 nw145 vdd vdd pch w=2u l=180n
CT146 t146 0 0.1f
M583 nw146 nd1 t146 0 nch w=1u l=180n
M584 t146 nw145 0 0 nch w=1u l=180n
Cnw146 nw146 0 2f
M585 nw147 nd2 vdd vdd pch w=2u l=180n
M586 nw147 nw145 vdd vdd pch w=2u l=180n
CT147 t147 0 0.1f
M587 nw147 nd2 t147 0 nch w=1u l=180n
M588 t147 nw145 0 0 nch w=1u l=180n
Cnw147 nw147 0 2f
M589 nw148 nw146 vdd vdd pch w=2u l=180n
M590 nw148 nw147 vdd vdd pch w=2u l=180n
CT148 t148 0 0.1f
M591 nw148 nw146 t148 0 nch w=1u l=180n
M592 t148 nw147 0 0 nch w=1u l=180n
Cnw148 nw148 0 2f
M593 nw149 nw148 vdd vdd pch w=2u l=180n
M594 nw149 nd3 vdd vdd pch w=2u l=180n
CT149 t149 0 0.1f
M595 nw149 nw148 t149 0 nch w=1u l=180n
M596 t149 nd3 0 0 nch w=1u l=180n
Cnw149 nw149 0 2f
M597 nw150 nw148 vdd vdd pch w=2u l=180n
M598 nw150 nw149 vdd vdd pch w=2u l=180n
CT150 t150 0 0.1f
M599 nw150 nw148 t150 0 nch w=1u l=180n
M600 t150 nw149 0 0 nch w=1u l=180n
Cnw150 nw150 0 2f
M601 nw151 nd3 vdd vdd pch w=2u l=180n
M602 nw151 nw149 vdd vdd pch w=2u l=180n
CT151 t151 0 0.1f
M603 nw151 nd3 t151 0 nch w=1u l=180n
M604 t151 nw149 0 0 nch w=1u l=180n
Cnw151 nw151 0 2f
M605 nw152 nw150 vdd vdd pch w=2u l=180n
M606 nw152 nw151 vdd vdd pch w=2u l=180n
CT152 t152 0 0.1f
M607 nw152 nw150 t152 0 nch w=1u l=180n
M608 t152 nw151 0 0 nch w=1u l=180n
Cnw152 nw152 0 2f
M609 nw153 nw152 vdd vdd pch w=2u l=180n
M610 nw153 nd7 vdd vdd pch w=2u l=180n
CT153 t153 0 0.1f
M611 nw153 nw152 t153 0 nch w=1u l=180n
M612 t153 nd7 0 0 nch w=1u l=180n
Cnw153 nw153 0 2f
M613 nw154 nw152 vdd vdd pch w=2u l=180n
M614 nw154 nw153 vdd vdd pch w=2u l=180n
CT154 t154 0 0.1f
M615 nw154 nw152 t154 0 nch w=1u l=180n
M616 t154 nw153 0 0 nch w=1u l=180n
Cnw154 nw154 0 2f
M617 nw155 nd7 vdd vdd pch w=2u l=180n
M618 nw155 nw153 vdd vdd pch w=2u l=180n
CT155 t155 0 0.1f
M619 nw155 nd7 t155 0 nch w=1u l=180n
M620 t155 nw153 0 0 nch w=1u l=180n
Cnw155 nw155 0 2f
M621 nw156 nw154 vdd vdd pch w=2u l=180n
M622 nw156 nw155 vdd vdd pch w=2u l=180n
CT156 t156 0 0.1f
M623 nw156 nw154 t156 0 nch w=1u l=180n
M624 t156 nw155 0 0 nch w=1u l=180n
Cnw156 nw156 0 2f
M625 nw157 nw156 vdd vdd pch w=2u l=180n
M626 nw157 nd8 vdd vdd pch w=2u l=180n
CT157 t157 0 0.1f
M627 nw157 nw156 t157 0 nch w=1u l=180n
M628 t157 nd8 0 0 nch w=1u l=180n
Cnw157 nw157 0 2f
M629 nw158 nw156 vdd vdd pch w=2u l=180n
M630 nw158 nw157 vdd vdd pch w=2u l=180n
CT158 t158 0 0.1f
M631 nw158 nw156 t158 0 nch w=1u l=180n
M632 t158 nw157 0 0 nch w=1u l=180n
Cnw158 nw158 0 2f
M633 nw159 nd8 vdd vdd pch w=2u l=180n
M634 nw159 nw157 vdd vdd pch w=2u l=180n
CT159 t159 0 0.1f
M635 nw159 nd8 t159 0 nch w=1u l=180n
M636 t159 nw157 0 0 nch w=1u l=180n
Cnw159 nw159 0 2f
M637 nw160 nw158 vdd vdd pch w=2u l=180n
M638 nw160 nw159 vdd vdd pch w=2u l=180n
CT160 t160 0 0.1f
M639 nw160 nw158 t160 0 nch w=1u l=180n
M640 t160 nw159 0 0 nch w=1u l=180n
Cnw160 nw160 0 2f
M641 nw161 nw160 vdd vdd pch w=2u l=180n
M642 nw161 nd9 vdd vdd pch w=2u l=180n
CT161 t161 0 0.1f
M643 nw161 nw160 t161 0 nch w=1u l=180n
M644 t161 nd9 0 0 nch w=1u l=180n
Cnw161 nw161 0 2f
M645 nw162 nw160 vdd vdd pch w=2u l=180n
M646 nw162 nw161 vdd vdd pch w=2u l=180n
CT162 t162 0 0.1f
M647 nw162 nw160 t162 0 nch w=1u l=180n
M648 t162 nw161 0 0 nch w=1u l=180n
Cnw162 nw162 0 2f
M649 nw163 nd9 vdd vdd pch w=2u l=180n
M650 nw163 nw161 vdd vdd pch w=2u l=180n
CT163 t163 0 0.1f
M651 nw163 nd9 t163 0 nch w=1u l=180n
M652 t163 nw161 0 0 nch w=1u l=180n
Cnw163 nw163 0 2f
M653 nw164 nw162 vdd vdd pch w=2u l=180n
M654 nw164 nw163 vdd vdd pch w=2u l=180n
CT164 t164 0 0.1f
M655 nw164 nw162 t164 0 nch w=1u l=180n
M656 t164 nw163 0 0 nch w=1u l=180n
Cnw164 nw164 0 2f
M657 nw165 nw164 vdd vdd pch w=2u l=180n
M658 nw165 nd10 vdd vdd pch w=2u l=180n
CT165 t165 0 0.1f
M659 nw165 nw164 t165 0 nch w=1u l=180n
M660 t165 nd10 0 0 nch w=1u l=180n
Cnw165 nw165 0 2f
M661 nw166 nw164 vdd vdd pch w=2u l=180n
M662 nw166 nw165 vdd vdd pch w=2u l=180n
CT166 t166 0 0.1f
M663 nw166 nw164 t166 0 nch w=1u l=180n
M664 t166 nw165 0 0 nch w=1u l=180n
Cnw166 nw166 0 2f
M665 nw167 nd10 vdd vdd pch w=2u l=180n
M666 nw167 nw165 vdd vdd pch w=2u l=180n
CT167 t167 0 0.1f
M667 nw167 nd10 t167 0 nch w=1u l=180n
M668 t167 nw165 0 0 nch w=1u l=180n
Cnw167 nw167 0 2f
M669 nw168 nw166 vdd vdd pch w=2u l=180n
M670 nw168 nw167 vdd vdd pch w=2u l=180n
CT168 t168 0 0.1f
M671 nw168 nw166 t168 0 nch w=1u l=180n
M672 t168 nw167 0 0 nch w=1u l=180n
Cnw168 nw168 0 2f
M673 nw169 nw168 vdd vdd pch w=2u l=180n
M674 nw169 nd14 vdd vdd pch w=2u l=180n
CT169 t169 0 0.1f
M675 nw169 nw168 t169 0 nch w=1u l=180n
M676 t169 nd14 0 0 nch w=1u l=180n
Cnw169 nw169 0 2f
M677 nw170 nw168 vdd vdd pch w=2u l=180n
M678 nw170 nw169 vdd vdd pch w=2u l=180n
CT170 t170 0 0.1f
M679 nw170 nw168 t170 0 nch w=1u l=180n
M680 t170 nw169 0 0 nch w=1u l=180n
Cnw170 nw170 0 2f
M681 nw171 nd14 vdd vdd pch w=2u l=180n
M682 nw171 nw169 vdd vdd pch w=2u l=180n
CT171 t171 0 0.1f
M683 nw171 nd14 t171 0 nch w=1u l=180n
M684 t171 nw169 0 0 nch w=1u l=180n
Cnw171 nw171 0 2f
M685 nw172 nw170 vdd vdd pch w=2u l=180n
M686 nw172 nw171 vdd vdd pch w=2u l=180n
CT172 t172 0 0.1f
M687 nw172 nw170 t172 0 nch w=1u l=180n
M688 t172 nw171 0 0 nch w=1u l=180n
Cnw172 nw172 0 2f
M689 nw173 nw172 vdd vdd pch w=2u l=180n
M690 nw173 nd15 vdd vdd pch w=2u l=180n
CT173 t173 0 0.1f
M691 nw173 nw172 t173 0 nch w=1u l=180n
M692 t173 nd15 0 0 nch w=1u l=180n
Cnw173 nw173 0 2f
M693 nw174 nw172 vdd vdd pch w=2u l=180n
M694 nw174 nw173 vdd vdd pch w=2u l=180n
CT174 t174 0 0.1f
M695 nw174 nw172 t174 0 nch w=1u l=180n
M696 t174 nw173 0 0 nch w=1u l=180n
Cnw174 nw174 0 2f
M697 nw175 nd15 vdd vdd pch w=2u l=180n
M698 nw175 nw173 vdd vdd pch w=2u l=180n
CT175 t175 0 0.1f
M699 nw175 nd15 t175 0 nch w=1u l=180n
M700 t175 nw173 0 0 nch w=1u l=180n
Cnw175 nw175 0 2f
M701 nw176 nw174 vdd vdd pch w=2u l=180n
M702 nw176 nw175 vdd vdd pch w=2u l=180n
CT176 t176 0 0.1f
M703 nw176 nw174 t176 0 nch w=1u l=180n
M704 t176 nw175 0 0 nch w=1u l=180n
Cnw176 nw176 0 2f
M705 nw177 nw176 vdd vdd pch w=2u l=180n
M706 nw177 nd16 vdd vdd pch w=2u l=180n
CT177 t177 0 0.1f
M707 nw177 nw176 t177 0 nch w=1u l=180n
M708 t177 nd16 0 0 nch w=1u l=180n
Cnw177 nw177 0 2f
M709 nw178 nw176 vdd vdd pch w=2u l=180n
M710 nw178 nw177 vdd vdd pch w=2u l=180n
CT178 t178 0 0.1f
M711 nw178 nw176 t178 0 nch w=1u l=180n
M712 t178 nw177 0 0 nch w=1u l=180n
Cnw178 nw178 0 2f
M713 nw179 nd16 vdd vdd pch w=2u l=180n
M714 nw179 nw177 vdd vdd pch w=2u l=180n
CT179 t179 0 0.1f
M715 nw179 nd16 t179 0 nch w=1u l=180n
M716 t179 nw177 0 0 nch w=1u l=180n
Cnw179 nw179 0 2f
M717 nw180 nw178 vdd vdd pch w=2u l=180n
M718 nw180 nw179 vdd vdd pch w=2u l=180n
CT180 t180 0 0.1f
M719 nw180 nw178 t180 0 nch w=1u l=180n
M720 t180 nw179 0 0 nch w=1u l=180n
Cnw180 nw180 0 2f
M721 nw181 nw180 vdd vdd pch w=2u l=180n
M722 nw181 nd17 vdd vdd pch w=2u l=180n
CT181 t181 0 0.1f
M723 nw181 nw180 t181 0 nch w=1u l=180n
M724 t181 nd17 0 0 nch w=1u l=180n
Cnw181 nw181 0 2f
M725 nw182 nw180 vdd vdd pch w=2u l=180n
M726 nw182 nw181 vdd vdd pch w=2u l=180n
CT182 t182 0 0.1f
M727 nw182 nw180 t182 0 nch w=1u l=180n
M728 t182 nw181 0 0 nch w=1u l=180n
Cnw182 nw182 0 2f
M729 nw183 nd17 vdd vdd pch w=2u l=180n
M730 nw183 nw181 vdd vdd pch w=2u l=180n
CT183 t183 0 0.1f
M731 nw183 nd17 t183 0 nch w=1u l=180n
M732 t183 nw181 0 0 nch w=1u l=180n
Cnw183 nw183 0 2f
M733 nw184 nw182 vdd vdd pch w=2u l=180n
M734 nw184 nw183 vdd vdd pch w=2u l=180n
CT184 t184 0 0.1f
M735 nw184 nw182 t184 0 nch w=1u l=180n
M736 t184 nw183 0 0 nch w=1u l=180n
Cnw184 nw184 0 2f
M737 nw185 nw184 vdd vdd pch w=2u l=180n
M738 nw185 nd22 vdd vdd pch w=2u l=180n
CT185 t185 0 0.1f
M739 nw185 nw184 t185 0 nch w=1u l=180n
M740 t185 nd22 0 0 nch w=1u l=180n
Cnw185 nw185 0 2f
M741 nw186 nw184 vdd vdd pch w=2u l=180n
M742 nw186 nw185 vdd vdd pch w=2u l=180n
CT186 t186 0 0.1f
M743 nw186 nw184 t186 0 nch w=1u l=180n
M744 t186 nw185 0 0 nch w=1u l=180n
Cnw186 nw186 0 2f
M745 nw187 nd22 vdd vdd pch w=2u l=180n
M746 nw187 nw185 vdd vdd pch w=2u l=180n
CT187 t187 0 0.1f
M747 nw187 nd22 t187 0 nch w=1u l=180n
M748 t187 nw185 0 0 nch w=1u l=180n
Cnw187 nw187 0 2f
M749 nw188 nw186 vdd vdd pch w=2u l=180n
M750 nw188 nw187 vdd vdd pch w=2u l=180n
CT188 t188 0 0.1f
M751 nw188 nw186 t188 0 nch w=1u l=180n
M752 t188 nw187 0 0 nch w=1u l=180n
Cnw188 nw188 0 2f
M753 nw189 nw188 vdd vdd pch w=2u l=180n
M754 nw189 nd23 vdd vdd pch w=2u l=180n
CT189 t189 0 0.1f
M755 nw189 nw188 t189 0 nch w=1u l=180n
M756 t189 nd23 0 0 nch w=1u l=180n
Cnw189 nw189 0 2f
M757 nw190 nw188 vdd vdd pch w=2u l=180n
M758 nw190 nw189 vdd vdd pch w=2u l=180n
CT190 t190 0 0.1f
M759 nw190 nw188 t190 0 nch w=1u l=180n
M760 t190 nw189 0 0 nch w=1u l=180n
Cnw190 nw190 0 2f
M761 nw191 nd23 vdd vdd pch w=2u l=180n
M762 nw191 nw189 vdd vdd pch w=2u l=180n
CT191 t191 0 0.1f
M763 nw191 nd23 t191 0 nch w=1u l=180n
M764 t191 nw189 0 0 nch w=1u l=180n
Cnw191 nw191 0 2f
M765 nw192 nw190 vdd vdd pch w=2u l=180n
M766 nw192 nw191 vdd vdd pch w=2u l=180n
CT192 t192 0 0.1f
M767 nw192 nw190 t192 0 nch w=1u l=180n
M768 t192 nw191 0 0 nch w=1u l=180n
Cnw192 nw192 0 2f
M769 nw193 nw192 vdd vdd pch w=2u l=180n
M770 nw193 nd24 vdd vdd pch w=2u l=180n
CT193 t193 0 0.1f
M771 nw193 nw192 t193 0 nch w=1u l=180n
M772 t193 nd24 0 0 nch w=1u l=180n
Cnw193 nw193 0 2f
M773 nw194 nw192 vdd vdd pch w=2u l=180n
M774 nw194 nw193 vdd vdd pch w=2u l=180n
CT194 t194 0 0.1f
M775 nw194 nw192 t194 0 nch w=1u l=180n
M776 t194 nw193 0 0 nch w=1u l=180n
Cnw194 nw194 0 2f
M777 nw195 nd24 vdd vdd pch w=2u l=180n
M778 nw195 nw193 vdd vdd pch w=2u l=180n
CT195 t195 0 0.1f
M779 nw195 nd24 t195 0 nch w=1u l=180n
M780 t195 nw193 0 0 nch w=1u l=180n
Cnw195 nw195 0 2f
M781 nw196 nw194 vdd vdd pch w=2u l=180n
M782 nw196 nw195 vdd vdd pch w=2u l=180n
CT196 t196 0 0.1f
M783 nw196 nw194 t196 0 nch w=1u l=180n
M784 t196 nw195 0 0 nch w=1u l=180n
Cnw196 nw196 0 2f
M785 nw197 nw196 vdd vdd pch w=2u l=180n
M786 nw197 nd25 vdd vdd pch w=2u l=180n
CT197 t197 0 0.1f
M787 nw197 nw196 t197 0 nch w=1u l=180n
M788 t197 nd25 0 0 nch w=1u l=180n
Cnw197 nw197 0 2f
M789 nw198 nw196 vdd vdd pch w=2u l=180n
M790 nw198 nw197 vdd vdd pch w=2u l=180n
CT198 t198 0 0.1f
M791 nw198 nw196 t198 0 nch w=1u l=180n
M792 t198 nw197 0 0 nch w=1u l=180n
Cnw198 nw198 0 2f
M793 nw199 nd25 vdd vdd pch w=2u l=180n
M794 nw199 nw197 vdd vdd pch w=2u l=180n
CT199 t199 0 0.1f
M795 nw199 nd25 t199 0 nch w=1u l=180n
M796 t199 nw197 0 0 nch w=1u l=180n
Cnw199 nw199 0 2f
M797 nw200 nw198 vdd vdd pch w=2u l=180n
M798 nw200 nw199 vdd vdd pch w=2u l=180n
CT200 t200 0 0.1f
M799 nw200 nw198 t200 0 nch w=1u l=180n
M800 t200 nw199 0 0 nch w=1u l=180n
Cnw200 nw200 0 2f
M801 nw201 nw200 vdd vdd pch w=2u l=180n
M802 nw201 nd29 vdd vdd pch w=2u l=180n
CT201 t201 0 0.1f
M803 nw201 nw200 t201 0 nch w=1u l=180n
M804 t201 nd29 0 0 nch w=1u l=180n
Cnw201 nw201 0 2f
M805 nw202 nw200 vdd vdd pch w=2u l=180n
M806 nw202 nw201 vdd vdd pch w=2u l=180n
CT202 t202 0 0.1f
M807 nw202 nw200 t202 0 nch w=1u l=180n
M808 t202 nw201 0 0 nch w=1u l=180n
Cnw202 nw202 0 2f
M809 nw203 nd29 vdd vdd pch w=2u l=180n
M810 nw203 nw201 vdd vdd pch w=2u l=180n
CT203 t203 0 0.1f
M811 nw203 nd29 t203 0 nch w=1u l=180n
M812 t203 nw201 0 0 nch w=1u l=180n
Cnw203 nw203 0 2f
M813 nw204 nw202 vdd vdd pch w=2u l=180n
M814 nw204 nw203 vdd vdd pch w=2u l=180n
CT204 t204 0 0.1f
M815 nw204 nw202 t204 0 nch w=1u l=180n
M816 t204 nw203 0 0 nch w=1u l=180n
Cnw204 nw204 0 2f
M817 nw205 nw204 vdd vdd pch w=2u l=180n
M818 nw205 nd30 vdd vdd pch w=2u l=180n
CT205 t205 0 0.1f
M819 nw205 nw204 t205 0 nch w=1u l=180n
M820 t205 nd30 0 0 nch w=1u l=180n
Cnw205 nw205 0 2f
M821 nw206 nw204 vdd vdd pch w=2u l=180n
M822 nw206 nw205 vdd vdd pch w=2u l=180n
CT206 t206 0 0.1f
M823 nw206 nw204 t206 0 nch w=1u l=180n
M824 t206 nw205 0 0 nch w=1u l=180n
Cnw206 nw206 0 2f
M825 nw207 nd30 vdd vdd pch w=2u l=180n
M826 nw207 nw205 vdd vdd pch w=2u l=180n
CT207 t207 0 0.1f
M827 nw207 nd30 t207 0 nch w=1u l=180n
M828 t207 nw205 0 0 nch w=1u l=180n
Cnw207 nw207 0 2f
M829 nw208 nw206 vdd vdd pch w=2u l=180n
M830 nw208 nw207 vdd vdd pch w=2u l=180n
CT208 t208 0 0.1f
M831 nw208 nw206 t208 0 nch w=1u l=180n
M832 t208 nw207 0 0 nch w=1u l=180n
Cnw208 nw208 0 2f
M833 nw209 nw208 vdd vdd pch w=2u l=180n
M834 nw209 nd31 vdd vdd pch w=2u l=180n
CT209 t209 0 0.1f
M835 nw209 nw208 t209 0 nch w=1u l=180n
M836 t209 nd31 0 0 nch w=1u l=180n
Cnw209 nw209 0 2f
M837 nw210 nw208 vdd vdd pch w=2u l=180n
M838 nw210 nw209 vdd vdd pch w=2u l=180n
CT210 t210 0 0.1f
M839 nw210 nw208 t210 0 nch w=1u l=180n
M840 t210 nw209 0 0 nch w=1u l=180n
Cnw210 nw210 0 2f
M841 nw211 nd31 vdd vdd pch w=2u l=180n
M842 nw211 nw209 vdd vdd pch w=2u l=180n
CT211 t211 0 0.1f
M843 nw211 nd31 t211 0 nch w=1u l=180n
M844 t211 nw209 0 0 nch w=1u l=180n
Cnw211 nw211 0 2f
M845 nw212 nw210 vdd vdd pch w=2u l=180n
M846 nw212 nw211 vdd vdd pch w=2u l=180n
CT212 t212 0 0.1f
M847 nw212 nw210 t212 0 nch w=1u l=180n
M848 t212 nw211 0 0 nch w=1u l=180n
Cnw212 nw212 0 2f
M849 nw213 nw212 vdd vdd pch w=2u l=180n
M850 nw213 nr2 vdd vdd pch w=2u l=180n
CT213 t213 0 0.1f
M851 nw213 nw212 t213 0 nch w=1u l=180n
M852 t213 nr2 0 0 nch w=1u l=180n
Cnw213 nw213 0 2f
M853 nw214 nw212 vdd vdd pch w=2u l=180n
M854 nw214 nw213 vdd vdd pch w=2u l=180n
CT214 t214 0 0.1f
M855 nw214 nw212 t214 0 nch w=1u l=180n
M856 t214 nw213 0 0 nch w=1u l=180n
Cnw214 nw214 0 2f
M857 nw215 nr2 vdd vdd pch w=2u l=180n
M858 nw215 nw213 vdd vdd pch w=2u l=180n
CT215 t215 0 0.1f
M859 nw215 nr2 t215 0 nch w=1u l=180n
M860 t215 nw213 0 0 nch w=1u l=180n
Cnw215 nw215 0 2f
M861 nw216 nw214 vdd vdd pch w=2u l=180n
M862 nw216 nw215 vdd vdd pch w=2u l=180n
CT216 t216 0 0.1f
M863 nw216 nw214 t216 0 nch w=1u l=180n
M864 t216 nw215 0 0 nch w=1u l=180n
Cnw216 nw216 0 2f
M865 nw217 nd4 vdd vdd pch w=2u l=180n
M866 nw217 nd5 vdd vdd pch w=2u l=180n
CT217 t217 0 0.1f
M867 nw217 nd4 t217 0 nch w=1u l=180n
M868 t217 nd5 0 0 nch w=1u l=180n
Cnw217 nw217 0 2f
M869 nw218 nd4 vdd vdd pch w=2u l=180n
M870 nw218 nw217 vdd vdd pch w=2u l=180n
CT218 t218 0 0.1f
M871 nw218 nd4 t218 0 nch w=1u l=180n
M872 t218 nw217 0 0 nch w=1u l=180n
Cnw218 nw218 0 2f
M873 nw219 nd5 vdd vdd pch w=2u l=180n
M874 nw219 nw217 vdd vdd pch w=2u l=180n
CT219 t219 0 0.1f
M875 nw219 nd5 t219 0 nch w=1u l=180n
M876 t219 nw217 0 0 nch w=1u l=180n
Cnw219 nw219 0 2f
M877 nw220 nw218 vdd vdd pch w=2u l=180n
M878 nw220 nw219 vdd vdd pch w=2u l=180n
CT220 t220 0 0.1f
M879 nw220 nw218 t220 0 nch w=1u l=180n
M880 t220 nw219 0 0 nch w=1u l=180n
Cnw220 nw220 0 2f
M881 nw221 nw220 vdd vdd pch w=2u l=180n
M882 nw221 nd6 vdd vdd pch w=2u l=180n
CT221 t221 0 0.1f
M883 nw221 nw220 t221 0 nch w=1u l=180n
M884 t221 nd6 0 0 nch w=1u l=180n
Cnw221 nw221 0 2f
M885 nw222 nw220 vdd vdd pch w=2u l=180n
M886 nw222 nw221 vdd vdd pch w=2u l=180n
CT222 t222 0 0.1f
M887 nw222 nw220 t222 0 nch w=1u l=180n
M888 t222 nw221 0 0 nch w=1u l=180n
Cnw222 nw222 0 2f
M889 nw223 nd6 vdd vdd pch w=2u l=180n
M890 nw223 nw221 vdd vdd pch w=2u l=180n
CT223 t223 0 0.1f
M891 nw223 nd6 t223 0 nch w=1u l=180n
M892 t223 nw221 0 0 nch w=1u l=180n
Cnw223 nw223 0 2f
M893 nw224 nw222 vdd vdd pch w=2u l=180n
M894 nw224 nw223 vdd vdd pch w=2u l=180n
CT224 t224 0 0.1f
M895 nw224 nw222 t224 0 nch w=1u l=180n
M896 t224 nw223 0 0 nch w=1u l=180n
Cnw224 nw224 0 2f
M897 nw225 nw224 vdd vdd pch w=2u l=180n
M898 nw225 nd7 vdd vdd pch w=2u l=180n
CT225 t225 0 0.1f
M899 nw225 nw224 t225 0 nch w=1u l=180n
M900 t225 nd7 0 0 nch w=1u l=180n
Cnw225 nw225 0 2f
M901 nw226 nw224 vdd vdd pch w=2u l=180n
M902 nw226 nw225 vdd vdd pch w=2u l=180n
CT226 t226 0 0.1f
M903 nw226 nw224 t226 0 nch w=1u l=180n
M904 t226 nw225 0 0 nch w=1u l=180n
Cnw226 nw226 0 2f
M905 nw227 nd7 vdd vdd pch w=2u l=180n
M906 nw227 nw225 vdd vdd pch w=2u l=180n
CT227 t227 0 0.1f
M907 nw227 nd7 t227 0 nch w=1u l=180n
M908 t227 nw225 0 0 nch w=1u l=180n
Cnw227 nw227 0 2f
M909 nw228 nw226 vdd vdd pch w=2u l=180n
M910 nw228 nw227 vdd vdd pch w=2u l=180n
CT228 t228 0 0.1f
M911 nw228 nw226 t228 0 nch w=1u l=180n
M912 t228 nw227 0 0 nch w=1u l=180n
Cnw228 nw228 0 2f
M913 nw229 nw228 vdd vdd pch w=2u l=180n
M914 nw229 nd8 vdd vdd pch w=2u l=180n
CT229 t229 0 0.1f
M915 nw229 nw228 t229 0 nch w=1u l=180n
M916 t229 nd8 0 0 nch w=1u l=180n
Cnw229 nw229 0 2f
M917 nw230 nw228 vdd vdd pch w=2u l=180n
M918 nw230 nw229 vdd vdd pch w=2u l=180n
CT230 t230 0 0.1f
M919 nw230 nw228 t230 0 nch w=1u l=180n
M920 t230 nw229 0 0 nch w=1u l=180n
Cnw230 nw230 0 2f
M921 nw231 nd8 vdd vdd pch w=2u l=180n
M922 nw231 nw229 vdd vdd pch w=2u l=180n
CT231 t231 0 0.1f
M923 nw231 nd8 t231 0 nch w=1u l=180n
M924 t231 nw229 0 0 nch w=1u l=180n
Cnw231 nw231 0 2f
M925 nw232 nw230 vdd vdd pch w=2u l=180n
M926 nw232 nw231 vdd vdd pch w=2u l=180n
CT232 t232 0 0.1f
M927 nw232 nw230 t232 0 nch w=1u l=180n
M928 t232 nw231 0 0 nch w=1u l=180n
Cnw232 nw232 0 2f
M929 nw233 nw232 vdd vdd pch w=2u l=180n
M930 nw233 nd9 vdd vdd pch w=2u l=180n
CT233 t233 0 0.1f
M931 nw233 nw232 t233 0 nch w=1u l=180n
M932 t233 nd9 0 0 nch w=1u l=180n
Cnw233 nw233 0 2f
M933 nw234 nw232 vdd vdd pch w=2u l=180n
M934 nw234 nw233 vdd vdd pch w=2u l=180n
CT234 t234 0 0.1f
M935 nw234 nw232 t234 0 nch w=1u l=180n
M936 t234 nw233 0 0 nch w=1u l=180n
Cnw234 nw234 0 2f
M937 nw235 nd9 vdd vdd pch w=2u l=180n
M938 nw235 nw233 vdd vdd pch w=2u l=180n
CT235 t235 0 0.1f
M939 nw235 nd9 t235 0 nch w=1u l=180n
M940 t235 nw233 0 0 nch w=1u l=180n
Cnw235 nw235 0 2f
M941 nw236 nw234 vdd vdd pch w=2u l=180n
M942 nw236 nw235 vdd vdd pch w=2u l=180n
CT236 t236 0 0.1f
M943 nw236 nw234 t236 0 nch w=1u l=180n
M944 t236 nw235 0 0 nch w=1u l=180n
Cnw236 nw236 0 2f
M945 nw237 nw236 vdd vdd pch w=2u l=180n
M946 nw237 nd10 vdd vdd pch w=2u l=180n
CT237 t237 0 0.1f
M947 nw237 nw236 t237 0 nch w=1u l=180n
M948 t237 nd10 0 0 nch w=1u l=180n
Cnw237 nw237 0 2f
M949 nw238 nw236 vdd vdd pch w=2u l=180n
M950 nw238 nw237 vdd vdd pch w=2u l=180n
CT238 t238 0 0.1f
M951 nw238 nw236 t238 0 nch w=1u l=180n
M952 t238 nw237 0 0 nch w=1u l=180n
Cnw238 nw238 0 2f
M953 nw239 nd10 vdd vdd pch w=2u l=180n
M954 nw239 nw237 vdd vdd pch w=2u l=180n
CT239 t239 0 0.1f
M955 nw239 nd10 t239 0 nch w=1u l=180n
M956 t239 nw237 0 0 nch w=1u l=180n
Cnw239 nw239 0 2f
M957 nw240 nw238 vdd vdd pch w=2u l=180n
M958 nw240 nw239 vdd vdd pch w=2u l=180n
CT240 t240 0 0.1f
M959 nw240 nw238 t240 0 nch w=1u l=180n
M960 t240 nw239 0 0 nch w=1u l=180n
Cnw240 nw240 0 2f
M961 nw241 nw240 vdd vdd pch w=2u l=180n
M962 nw241 nd18 vdd vdd pch w=2u l=180n
CT241 t241 0 0.1f
M963 nw241 nw240 t241 0 nch w=1u l=180n
M964 t241 nd18 0 0 nch w=1u l=180n
Cnw241 nw241 0 2f
M965 nw242 nw240 vdd vdd pch w=2u l=180n
M966 nw242 nw241 vdd vdd pch w=2u l=180n
CT242 t242 0 0.1f
M967 nw242 nw240 t242 0 nch w=1u l=180n
M968 t242 nw241 0 0 nch w=1u l=180n
Cnw242 nw242 0 2f
M969 nw243 nd18 vdd vdd pch w=2u l=180n
M970 nw243 nw241 vdd vdd pch w=2u l=180n
CT243 t243 0 0.1f
M971 nw243 nd18 t243 0 nch w=1u l=180n
M972 t243 nw241 0 0 nch w=1u l=180n
Cnw243 nw243 0 2f
M973 nw244 nw242 vdd vdd pch w=2u l=180n
M974 nw244 nw243 vdd vdd pch w=2u l=180n
CT244 t244 0 0.1f
M975 nw244 nw242 t244 0 nch w=1u l=180n
M976 t244 nw243 0 0 nch w=1u l=180n
Cnw244 nw244 0 2f
M977 nw245 nw244 vdd vdd pch w=2u l=180n
M978 nw245 nd19 vdd vdd pch w=2u l=180n
CT245 t245 0 0.1f
M979 nw245 nw244 t245 0 nch w=1u l=180n
M980 t245 nd19 0 0 nch w=1u l=180n
Cnw245 nw245 0 2f
M981 nw246 nw244 vdd vdd pch w=2u l=180n
M982 nw246 nw245 vdd vdd pch w=2u l=180n
CT246 t246 0 0.1f
M983 nw246 nw244 t246 0 nch w=1u l=180n
M984 t246 nw245 0 0 nch w=1u l=180n
Cnw246 nw246 0 2f
M985 nw247 nd19 vdd vdd pch w=2u l=180n
M986 nw247 nw245 vdd vdd pch w=2u l=180n
CT247 t247 0 0.1f
M987 nw247 nd19 t247 0 nch w=1u l=180n
M988 t247 nw245 0 0 nch w=1u l=180n
Cnw247 nw247 0 2f
M989 nw248 nw246 vdd vdd pch w=2u l=180n
M990 nw248 nw247 vdd vdd pch w=2u l=180n
CT248 t248 0 0.1f
M991 nw248 nw246 t248 0 nch w=1u l=180n
M992 t248 nw247 0 0 nch w=1u l=180n
Cnw248 nw248 0 2f
M993 nw249 nw248 vdd vdd pch w=2u l=180n
M994 nw249 nd20 vdd vdd pch w=2u l=180n
CT249 t249 0 0.1f
M995 nw249 nw248 t249 0 nch w=1u l=180n
M996 t249 nd20 0 0 nch w=1u l=180n
Cnw249 nw249 0 2f
M997 nw250 nw248 vdd vdd pch w=2u l=180n
M998 nw250 nw249 vdd vdd pch w=2u l=180n
CT250 t250 0 0.1f
M999 nw250 nw248 t250 0 nch w=1u l=180n
M1000 t250 nw249 0 0 nch w=1u l=180n
Cnw250 nw250 0 2f
M1001 nw251 nd20 vdd vdd pch w=2u l=180n
M1002 nw251 nw249 vdd vdd pch w=2u l=180n
CT251 t251 0 0.1f
M1003 nw251 nd20 t251 0 nch w=1u l=180n
M1004 t251 nw249 0 0 nch w=1u l=180n
Cnw251 nw251 0 2f
M1005 nw252 nw250 vdd vdd pch w=2u l=180n
M1006 nw252 nw251 vdd vdd pch w=2u l=180n
CT252 t252 0 0.1f
M1007 nw252 nw250 t252 0 nch w=1u l=180n
M1008 t252 nw251 0 0 nch w=1u l=180n
Cnw252 nw252 0 2f
M1009 nw253 nw252 vdd vdd pch w=2u l=180n
M1010 nw253 nd21 vdd vdd pch w=2u l=180n
CT253 t253 0 0.1f
M1011 nw253 nw252 t253 0 nch w=1u l=180n
M1012 t253 nd21 0 0 nch w=1u l=180n
Cnw253 nw253 0 2f
M1013 nw254 nw252 vdd vdd pch w=2u l=180n
M1014 nw254 nw253 vdd vdd pch w=2u l=180n
CT254 t254 0 0.1f
M1015 nw254 nw252 t254 0 nch w=1u l=180n
M1016 t254 nw253 0 0 nch w=1u l=180n
Cnw254 nw254 0 2f
M1017 nw255 nd21 vdd vdd pch w=2u l=180n
M1018 nw255 nw253 vdd vdd pch w=2u l=180n
CT255 t255 0 0.1f
M1019 nw255 nd21 t255 0 nch w=1u l=180n
M1020 t255 nw253 0 0 nch w=1u l=180n
Cnw255 nw255 0 2f
M1021 nw256 nw254 vdd vdd pch w=2u l=180n
M1022 nw256 nw255 vdd vdd pch w=2u l=180n
CT256 t256 0 0.1f
M1023 nw256 nw254 t256 0 nch w=1u l=180n
M1024 t256 nw255 0 0 nch w=1u l=180n
Cnw256 nw256 0 2f
M1025 nw257 nw256 vdd vdd pch w=2u l=180n
M1026 nw257 nd22 vdd vdd pch w=2u l=180n
CT257 t257 0 0.1f
M1027 nw257 nw256 t257 0 nch w=1u l=180n
M1028 t257 nd22 0 0 nch w=1u l=180n
Cnw257 nw257 0 2f
M1029 nw258 nw256 vdd vdd pch w=2u l=180n
M1030 nw258 nw257 vdd vdd pch w=2u l=180n
CT258 t258 0 0.1f
M1031 nw258 nw256 t258 0 nch w=1u l=180n
M1032 t258 nw257 0 0 nch w=1u l=180n
Cnw258 nw258 0 2f
M1033 nw259 nd22 vdd vdd pch w=2u l=180n
M1034 nw259 nw257 vdd vdd pch w=2u l=180n
CT259 t259 0 0.1f
M1035 nw259 nd22 t259 0 nch w=1u l=180n
M1036 t259 nw257 0 0 nch w=1u l=180n
Cnw259 nw259 0 2f
M1037 nw260 nw258 vdd vdd pch w=2u l=180n
M1038 nw260 nw259 vdd vdd pch w=2u l=180n
CT260 t260 0 0.1f
M1039 nw260 nw258 t260 0 nch w=1u l=180n
M1040 t260 nw259 0 0 nch w=1u l=180n
Cnw260 nw260 0 2f
M1041 nw261 nw260 vdd vdd pch w=2u l=180n
M1042 nw261 nd23 vdd vdd pch w=2u l=180n
CT261 t261 0 0.1f
M1043 nw261 nw260 t261 0 nch w=1u l=180n
M1044 t261 nd23 0 0 nch w=1u l=180n
Cnw261 nw261 0 2f
M1045 nw262 nw260 vdd vdd pch w=2u l=180n
M1046 nw262 nw261 vdd vdd pch w=2u l=180n
CT262 t262 0 0.1f
M1047 nw262 nw260 t262 0 nch w=1u l=180n
M1048 t262 nw261 0 0 nch w=1u l=180n
Cnw262 nw262 0 2f
M1049 nw263 nd23 vdd vdd pch w=2u l=180n
M1050 nw263 nw261 vdd vdd pch w=2u l=180n
CT263 t263 0 0.1f
M1051 nw263 nd23 t263 0 nch w=1u l=180n
M1052 t263 nw261 0 0 nch w=1u l=180n
Cnw263 nw263 0 2f
M1053 nw264 nw262 vdd vdd pch w=2u l=180n
M1054 nw264 nw263 vdd vdd pch w=2u l=180n
CT264 t264 0 0.1f
M1055 nw264 nw262 t264 0 nch w=1u l=180n
M1056 t264 nw263 0 0 nch w=1u l=180n
Cnw264 nw264 0 2f
M1057 nw265 nw264 vdd vdd pch w=2u l=180n
M1058 nw265 nd24 vdd vdd pch w=2u l=180n
CT265 t265 0 0.1f
M1059 nw265 nw264 t265 0 nch w=1u l=180n
M1060 t265 nd24 0 0 nch w=1u l=180n
Cnw265 nw265 0 2f
M1061 nw266 nw264 vdd vdd pch w=2u l=180n
M1062 nw266 nw265 vdd vdd pch w=2u l=180n
CT266 t266 0 0.1f
M1063 nw266 nw264 t266 0 nch w=1u l=180n
M1064 t266 nw265 0 0 nch w=1u l=180n
Cnw266 nw266 0 2f
M1065 nw267 nd24 vdd vdd pch w=2u l=180n
M1066 nw267 nw265 vdd vdd pch w=2u l=180n
CT267 t267 0 0.1f
M1067 nw267 nd24 t267 0 nch w=1u l=180n
M1068 t267 nw265 0 0 nch w=1u l=180n
Cnw267 nw267 0 2f
M1069 nw268 nw266 vdd vdd pch w=2u l=180n
M1070 nw268 nw267 vdd vdd pch w=2u l=180n
CT268 t268 0 0.1f
M1071 nw268 nw266 t268 0 nch w=1u l=180n
M1072 t268 nw267 0 0 nch w=1u l=180n
Cnw268 nw268 0 2f
M1073 nw269 nw268 vdd vdd pch w=2u l=180n
M1074 nw269 nd25 vdd vdd pch w=2u l=180n
CT269 t269 0 0.1f
M1075 nw269 nw268 t269 0 nch w=1u l=180n
M1076 t269 nd25 0 0 nch w=1u l=180n
Cnw269 nw269 0 2f
M1077 nw270 nw268 vdd vdd pch w=2u l=180n
M1078 nw270 nw269 vdd vdd pch w=2u l=180n
CT270 t270 0 0.1f
M1079 nw270 nw268 t270 0 nch w=1u l=180n
M1080 t270 nw269 0 0 nch w=1u l=180n
Cnw270 nw270 0 2f
M1081 nw271 nd25 vdd vdd pch w=2u l=180n
M1082 nw271 nw269 vdd vdd pch w=2u l=180n
CT271 t271 0 0.1f
M1083 nw271 nd25 t271 0 nch w=1u l=180n
M1084 t271 nw269 0 0 nch w=1u l=180n
Cnw271 nw271 0 2f
M1085 nw272 nw270 vdd vdd pch w=2u l=180n
M1086 nw272 nw271 vdd vdd pch w=2u l=180n
CT272 t272 0 0.1f
M1087 nw272 nw270 t272 0 nch w=1u l=180n
M1088 t272 nw271 0 0 nch w=1u l=180n
Cnw272 nw272 0 2f
M1089 nw273 nw272 vdd vdd pch w=2u l=180n
M1090 nw273 nr3 vdd vdd pch w=2u l=180n
CT273 t273 0 0.1f
M1091 nw273 nw272 t273 0 nch w=1u l=180n
M1092 t273 nr3 0 0 nch w=1u l=180n
Cnw273 nw273 0 2f
M1093 nw274 nw272 vdd vdd pch w=2u l=180n
M1094 nw274 nw273 vdd vdd pch w=2u l=180n
CT274 t274 0 0.1f
M1095 nw274 nw272 t274 0 nch w=1u l=180n
M1096 t274 nw273 0 0 nch w=1u l=180n
Cnw274 nw274 0 2f
M1097 nw275 nr3 vdd vdd pch w=2u l=180n
M1098 nw275 nw273 vdd vdd pch w=2u l=180n
CT275 t275 0 0.1f
M1099 nw275 nr3 t275 0 nch w=1u l=180n
M1100 t275 nw273 0 0 nch w=1u l=180n
Cnw275 nw275 0 2f
M1101 nw276 nw274 vdd vdd pch w=2u l=180n
M1102 nw276 nw275 vdd vdd pch w=2u l=180n
CT276 t276 0 0.1f
M1103 nw276 nw274 t276 0 nch w=1u l=180n
M1104 t276 nw275 0 0 nch w=1u l=180n
Cnw276 nw276 0 2f
M1105 nw277 nd11 vdd vdd pch w=2u l=180n
M1106 nw277 nd12 vdd vdd pch w=2u l=180n
CT277 t277 0 0.1f
M1107 nw277 nd11 t277 0 nch w=1u l=180n
M1108 t277 nd12 0 0 nch w=1u l=180n
Cnw277 nw277 0 2f
M1109 nw278 nd11 vdd vdd pch w=2u l=180n
M1110 nw278 nw277 vdd vdd pch w=2u l=180n
CT278 t278 0 0.1f
M1111 nw278 nd11 t278 0 nch w=1u l=180n
M1112 t278 nw277 0 0 nch w=1u l=180n
Cnw278 nw278 0 2f
M1113 nw279 nd12 vdd vdd pch w=2u l=180n
M1114 nw279 nw277 vdd vdd pch w=2u l=180n
CT279 t279 0 0.1f
M1115 nw279 nd12 t279 0 nch w=1u l=180n
M1116 t279 nw277 0 0 nch w=1u l=180n
Cnw279 nw279 0 2f
M1117 nw280 nw278 vdd vdd pch w=2u l=180n
M1118 nw280 nw279 vdd vdd pch w=2u l=180n
CT280 t280 0 0.1f
M1119 nw280 nw278 t280 0 nch w=1u l=180n
M1120 t280 nw279 0 0 nch w=1u l=180n
Cnw280 nw280 0 2f
M1121 nw281 nw280 vdd vdd pch w=2u l=180n
M1122 nw281 nd13 vdd vdd pch w=2u l=180n
CT281 t281 0 0.1f
M1123 nw281 nw280 t281 0 nch w=1u l=180n
M1124 t281 nd13 0 0 nch w=1u l=180n
Cnw281 nw281 0 2f
M1125 nw282 nw280 vdd vdd pch w=2u l=180n
M1126 nw282 nw281 vdd vdd pch w=2u l=180n
CT282 t282 0 0.1f
M1127 nw282 nw280 t282 0 nch w=1u l=180n
M1128 t282 nw281 0 0 nch w=1u l=180n
Cnw282 nw282 0 2f
M1129 nw283 nd13 vdd vdd pch w=2u l=180n
M1130 nw283 nw281 vdd vdd pch w=2u l=180n
CT283 t283 0 0.1f
M1131 nw283 nd13 t283 0 nch w=1u l=180n
M1132 t283 nw281 0 0 nch w=1u l=180n
Cnw283 nw283 0 2f
M1133 nw284 nw282 vdd vdd pch w=2u l=180n
M1134 nw284 nw283 vdd vdd pch w=2u l=180n
CT284 t284 0 0.1f
M1135 nw284 nw282 t284 0 nch w=1u l=180n
M1136 t284 nw283 0 0 nch w=1u l=180n
Cnw284 nw284 0 2f
M1137 nw285 nw284 vdd vdd pch w=2u l=180n
M1138 nw285 nd14 vdd vdd pch w=2u l=180n
CT285 t285 0 0.1f
M1139 nw285 nw284 t285 0 nch w=1u l=180n
M1140 t285 nd14 0 0 nch w=1u l=180n
Cnw285 nw285 0 2f
M1141 nw286 nw284 vdd vdd pch w=2u l=180n
M1142 nw286 nw285 vdd vdd pch w=2u l=180n
CT286 t286 0 0.1f
M1143 nw286 nw284 t286 0 nch w=1u l=180n
M1144 t286 nw285 0 0 nch w=1u l=180n
Cnw286 nw286 0 2f
M1145 nw287 nd14 vdd vdd pch w=2u l=180n
M1146 nw287 nw285 vdd vdd pch w=2u l=180n
CT287 t287 0 0.1f
M1147 nw287 nd14 t287 0 nch w=1u l=180n
M1148 t287 nw285 0 0 nch w=1u l=180n
Cnw287 nw287 0 2f
M1149 nw288 nw286 vdd vdd pch w=2u l=180n
M1150 nw288 nw287 vdd vdd pch w=2u l=180n
CT288 t288 0 0.1f
M1151 nw288 nw286 t288 0 nch w=1u l=180n
M1152 t288 nw287 0 0 nch w=1u l=180n
Cnw288 nw288 0 2f
M1153 nw289 nw288 vdd vdd pch w=2u l=180n
M1154 nw289 nd15 vdd vdd pch w=2u l=180n
CT289 t289 0 0.1f
M1155 nw289 nw288 t289 0 nch w=1u l=180n
M1156 t289 nd15 0 0 nch w=1u l=180n
Cnw289 nw289 0 2f
M1157 nw290 nw288 vdd vdd pch w=2u l=180n
M1158 nw290 nw289 vdd vdd pch w=2u l=180n
CT290 t290 0 0.1f
M1159 nw290 nw288 t290 0 nch w=1u l=180n
M1160 t290 nw289 0 0 nch w=1u l=180n
Cnw290 nw290 0 2f
M1161 nw291 nd15 vdd vdd pch w=2u l=180n
M1162 nw291 nw289 vdd vdd pch w=2u l=180n
CT291 t291 0 0.1f
M1163 nw291 nd15 t291 0 nch w=1u l=180n
M1164 t291 nw289 0 0 nch w=1u l=180n
Cnw291 nw291 0 2f
M1165 nw292 nw290 vdd vdd pch w=2u l=180n
M1166 nw292 nw291 vdd vdd pch w=2u l=180n
CT292 t292 0 0.1f
M1167 nw292 nw290 t292 0 nch w=1u l=180n
M1168 t292 nw291 0 0 nch w=1u l=180n
Cnw292 nw292 0 2f
M1169 nw293 nw292 vdd vdd pch w=2u l=180n
M1170 nw293 nd16 vdd vdd pch w=2u l=180n
CT293 t293 0 0.1f
M1171 nw293 nw292 t293 0 nch w=1u l=180n
M1172 t293 nd16 0 0 nch w=1u l=180n
Cnw293 nw293 0 2f
M1173 nw294 nw292 vdd vdd pch w=2u l=180n
M1174 nw294 nw293 vdd vdd pch w=2u l=180n
CT294 t294 0 0.1f
M1175 nw294 nw292 t294 0 nch w=1u l=180n
M1176 t294 nw293 0 0 nch w=1u l=180n
Cnw294 nw294 0 2f
M1177 nw295 nd16 vdd vdd pch w=2u l=180n
M1178 nw295 nw293 vdd vdd pch w=2u l=180n
CT295 t295 0 0.1f
M1179 nw295 nd16 t295 0 nch w=1u l=180n
M1180 t295 nw293 0 0 nch w=1u l=180n
Cnw295 nw295 0 2f
M1181 nw296 nw294 vdd vdd pch w=2u l=180n
M1182 nw296 nw295 vdd vdd pch w=2u l=180n
CT296 t296 0 0.1f
M1183 nw296 nw294 t296 0 nch w=1u l=180n
M1184 t296 nw295 0 0 nch w=1u l=180n
Cnw296 nw296 0 2f
M1185 nw297 nw296 vdd vdd pch w=2u l=180n
M1186 nw297 nd17 vdd vdd pch w=2u l=180n
CT297 t297 0 0.1f
M1187 nw297 nw296 t297 0 nch w=1u l=180n
M1188 t297 nd17 0 0 nch w=1u l=180n
Cnw297 nw297 0 2f
M1189 nw298 nw296 vdd vdd pch w=2u l=180n
M1190 nw298 nw297 vdd vdd pch w=2u l=180n
CT298 t298 0 0.1f
M1191 nw298 nw296 t298 0 nch w=1u l=180n
M1192 t298 nw297 0 0 nch w=1u l=180n
Cnw298 nw298 0 2f
M1193 nw299 nd17 vdd vdd pch w=2u l=180n
M1194 nw299 nw297 vdd vdd pch w=2u l=180n
CT299 t299 0 0.1f
M1195 nw299 nd17 t299 0 nch w=1u l=180n
M1196 t299 nw297 0 0 nch w=1u l=180n
Cnw299 nw299 0 2f
M1197 nw300 nw298 vdd vdd pch w=2u l=180n
M1198 nw300 nw299 vdd vdd pch w=2u l=180n
CT300 t300 0 0.1f
M1199 nw300 nw298 t300 0 nch w=1u l=180n
M1200 t300 nw299 0 0 nch w=1u l=180n
Cnw300 nw300 0 2f
M1201 nw301 nw300 vdd vdd pch w=2u l=180n
M1202 nw301 nd18 vdd vdd pch w=2u l=180n
CT301 t301 0 0.1f
M1203 nw301 nw300 t301 0 nch w=1u l=180n
M1204 t301 nd18 0 0 nch w=1u l=180n
Cnw301 nw301 0 2f
M1205 nw302 nw300 vdd vdd pch w=2u l=180n
M1206 nw302 nw301 vdd vdd pch w=2u l=180n
CT302 t302 0 0.1f
M1207 nw302 nw300 t302 0 nch w=1u l=180n
M1208 t302 nw301 0 0 nch w=1u l=180n
Cnw302 nw302 0 2f
M1209 nw303 nd18 vdd vdd pch w=2u l=180n
M1210 nw303 nw301 vdd vdd pch w=2u l=180n
CT303 t303 0 0.1f
M1211 nw303 nd18 t303 0 nch w=1u l=180n
M1212 t303 nw301 0 0 nch w=1u l=180n
Cnw303 nw303 0 2f
M1213 nw304 nw302 vdd vdd pch w=2u l=180n
M1214 nw304 nw303 vdd vdd pch w=2u l=180n
CT304 t304 0 0.1f
M1215 nw304 nw302 t304 0 nch w=1u l=180n
M1216 t304 nw303 0 0 nch w=1u l=180n
Cnw304 nw304 0 2f
M1217 nw305 nw304 vdd vdd pch w=2u l=180n
M1218 nw305 nd19 vdd vdd pch w=2u l=180n
CT305 t305 0 0.1f
M1219 nw305 nw304 t305 0 nch w=1u l=180n
M1220 t305 nd19 0 0 nch w=1u l=180n
Cnw305 nw305 0 2f
M1221 nw306 nw304 vdd vdd pch w=2u l=180n
M1222 nw306 nw305 vdd vdd pch w=2u l=180n
CT306 t306 0 0.1f
M1223 nw306 nw304 t306 0 nch w=1u l=180n
M1224 t306 nw305 0 0 nch w=1u l=180n
Cnw306 nw306 0 2f
M1225 nw307 nd19 vdd vdd pch w=2u l=180n
M1226 nw307 nw305 vdd vdd pch w=2u l=180n
CT307 t307 0 0.1f
M1227 nw307 nd19 t307 0 nch w=1u l=180n
M1228 t307 nw305 0 0 nch w=1u l=180n
Cnw307 nw307 0 2f
M1229 nw308 nw306 vdd vdd pch w=2u l=180n
M1230 nw308 nw307 vdd vdd pch w=2u l=180n
CT308 t308 0 0.1f
M1231 nw308 nw306 t308 0 nch w=1u l=180n
M1232 t308 nw307 0 0 nch w=1u l=180n
Cnw308 nw308 0 2f
M1233 nw309 nw308 vdd vdd pch w=2u l=180n
M1234 nw309 nd20 vdd vdd pch w=2u l=180n
CT309 t309 0 0.1f
M1235 nw309 nw308 t309 0 nch w=1u l=180n
M1236 t309 nd20 0 0 nch w=1u l=180n
Cnw309 nw309 0 2f
M1237 nw310 nw308 vdd vdd pch w=2u l=180n
M1238 nw310 nw309 vdd vdd pch w=2u l=180n
CT310 t310 0 0.1f
M1239 nw310 nw308 t310 0 nch w=1u l=180n
M1240 t310 nw309 0 0 nch w=1u l=180n
Cnw310 nw310 0 2f
M1241 nw311 nd20 vdd vdd pch w=2u l=180n
M1242 nw311 nw309 vdd vdd pch w=2u l=180n
CT311 t311 0 0.1f
M1243 nw311 nd20 t311 0 nch w=1u l=180n
M1244 t311 nw309 0 0 nch w=1u l=180n
Cnw311 nw311 0 2f
M1245 nw312 nw310 vdd vdd pch w=2u l=180n
M1246 nw312 nw311 vdd vdd pch w=2u l=180n
CT312 t312 0 0.1f
M1247 nw312 nw310 t312 0 nch w=1u l=180n
M1248 t312 nw311 0 0 nch w=1u l=180n
Cnw312 nw312 0 2f
M1249 nw313 nw312 vdd vdd pch w=2u l=180n
M1250 nw313 nd21 vdd vdd pch w=2u l=180n
CT313 t313 0 0.1f
M1251 nw313 nw312 t313 0 nch w=1u l=180n
M1252 t313 nd21 0 0 nch w=1u l=180n
Cnw313 nw313 0 2f
M1253 nw314 nw312 vdd vdd pch w=2u l=180n
M1254 nw314 nw313 vdd vdd pch w=2u l=180n
CT314 t314 0 0.1f
M1255 nw314 nw312 t314 0 nch w=1u l=180n
M1256 t314 nw313 0 0 nch w=1u l=180n
Cnw314 nw314 0 2f
M1257 nw315 nd21 vdd vdd pch w=2u l=180n
M1258 nw315 nw313 vdd vdd pch w=2u l=180n
CT315 t315 0 0.1f
M1259 nw315 nd21 t315 0 nch w=1u l=180n
M1260 t315 nw313 0 0 nch w=1u l=180n
Cnw315 nw315 0 2f
M1261 nw316 nw314 vdd vdd pch w=2u l=180n
M1262 nw316 nw315 vdd vdd pch w=2u l=180n
CT316 t316 0 0.1f
M1263 nw316 nw314 t316 0 nch w=1u l=180n
M1264 t316 nw315 0 0 nch w=1u l=180n
Cnw316 nw316 0 2f
M1265 nw317 nw316 vdd vdd pch w=2u l=180n
M1266 nw317 nd22 vdd vdd pch w=2u l=180n
CT317 t317 0 0.1f
M1267 nw317 nw316 t317 0 nch w=1u l=180n
M1268 t317 nd22 0 0 nch w=1u l=180n
Cnw317 nw317 0 2f
M1269 nw318 nw316 vdd vdd pch w=2u l=180n
M1270 nw318 nw317 vdd vdd pch w=2u l=180n
CT318 t318 0 0.1f
M1271 nw318 nw316 t318 0 nch w=1u l=180n
M1272 t318 nw317 0 0 nch w=1u l=180n
Cnw318 nw318 0 2f
M1273 nw319 nd22 vdd vdd pch w=2u l=180n
M1274 nw319 nw317 vdd vdd pch w=2u l=180n
CT319 t319 0 0.1f
M1275 nw319 nd22 t319 0 nch w=1u l=180n
M1276 t319 nw317 0 0 nch w=1u l=180n
Cnw319 nw319 0 2f
M1277 nw320 nw318 vdd vdd pch w=2u l=180n
M1278 nw320 nw319 vdd vdd pch w=2u l=180n
CT320 t320 0 0.1f
M1279 nw320 nw318 t320 0 nch w=1u l=180n
M1280 t320 nw319 0 0 nch w=1u l=180n
Cnw320 nw320 0 2f
M1281 nw321 nw320 vdd vdd pch w=2u l=180n
M1282 nw321 nd23 vdd vdd pch w=2u l=180n
CT321 t321 0 0.1f
M1283 nw321 nw320 t321 0 nch w=1u l=180n
M1284 t321 nd23 0 0 nch w=1u l=180n
Cnw321 nw321 0 2f
M1285 nw322 nw320 vdd vdd pch w=2u l=180n
M1286 nw322 nw321 vdd vdd pch w=2u l=180n
CT322 t322 0 0.1f
M1287 nw322 nw320 t322 0 nch w=1u l=180n
M1288 t322 nw321 0 0 nch w=1u l=180n
Cnw322 nw322 0 2f
M1289 nw323 nd23 vdd vdd pch w=2u l=180n
M1290 nw323 nw321 vdd vdd pch w=2u l=180n
CT323 t323 0 0.1f
M1291 nw323 nd23 t323 0 nch w=1u l=180n
M1292 t323 nw321 0 0 nch w=1u l=180n
Cnw323 nw323 0 2f
M1293 nw324 nw322 vdd vdd pch w=2u l=180n
M1294 nw324 nw323 vdd vdd pch w=2u l=180n
CT324 t324 0 0.1f
M1295 nw324 nw322 t324 0 nch w=1u l=180n
M1296 t324 nw323 0 0 nch w=1u l=180n
Cnw324 nw324 0 2f
M1297 nw325 nw324 vdd vdd pch w=2u l=180n
M1298 nw325 nd24 vdd vdd pch w=2u l=180n
CT325 t325 0 0.1f
M1299 nw325 nw324 t325 0 nch w=1u l=180n
M1300 t325 nd24 0 0 nch w=1u l=180n
Cnw325 nw325 0 2f
M1301 nw326 nw324 vdd vdd pch w=2u l=180n
M1302 nw326 nw325 vdd vdd pch w=2u l=180n
CT326 t326 0 0.1f
M1303 nw326 nw324 t326 0 nch w=1u l=180n
M1304 t326 nw325 0 0 nch w=1u l=180n
Cnw326 nw326 0 2f
M1305 nw327 nd24 vdd vdd pch w=2u l=180n
M1306 nw327 nw325 vdd vdd pch w=2u l=180n
CT327 t327 0 0.1f
M1307 nw327 nd24 t327 0 nch w=1u l=180n
M1308 t327 nw325 0 0 nch w=1u l=180n
Cnw327 nw327 0 2f
M1309 nw328 nw326 vdd vdd pch w=2u l=180n
M1310 nw328 nw327 vdd vdd pch w=2u l=180n
CT328 t328 0 0.1f
M1311 nw328 nw326 t328 0 nch w=1u l=180n
M1312 t328 nw327 0 0 nch w=1u l=180n
Cnw328 nw328 0 2f
M1313 nw329 nw328 vdd vdd pch w=2u l=180n
M1314 nw329 nd25 vdd vdd pch w=2u l=180n
CT329 t329 0 0.1f
M1315 nw329 nw328 t329 0 nch w=1u l=180n
M1316 t329 nd25 0 0 nch w=1u l=180n
Cnw329 nw329 0 2f
M1317 nw330 nw328 vdd vdd pch w=2u l=180n
M1318 nw330 nw329 vdd vdd pch w=2u l=180n
CT330 t330 0 0.1f
M1319 nw330 nw328 t330 0 nch w=1u l=180n
M1320 t330 nw329 0 0 nch w=1u l=180n
Cnw330 nw330 0 2f
M1321 nw331 nd25 vdd vdd pch w=2u l=180n
M1322 nw331 nw329 vdd vdd pch w=2u l=180n
CT331 t331 0 0.1f
M1323 nw331 nd25 t331 0 nch w=1u l=180n
M1324 t331 nw329 0 0 nch w=1u l=180n
Cnw331 nw331 0 2f
M1325 nw332 nw330 vdd vdd pch w=2u l=180n
M1326 nw332 nw331 vdd vdd pch w=2u l=180n
CT332 t332 0 0.1f
M1327 nw332 nw330 t332 0 nch w=1u l=180n
M1328 t332 nw331 0 0 nch w=1u l=180n
Cnw332 nw332 0 2f
M1329 nw333 nw332 vdd vdd pch w=2u l=180n
M1330 nw333 nr4 vdd vdd pch w=2u l=180n
CT333 t333 0 0.1f
M1331 nw333 nw332 t333 0 nch w=1u l=180n
M1332 t333 nr4 0 0 nch w=1u l=180n
Cnw333 nw333 0 2f
M1333 nw334 nw332 vdd vdd pch w=2u l=180n
M1334 nw334 nw333 vdd vdd pch w=2u l=180n
CT334 t334 0 0.1f
M1335 nw334 nw332 t334 0 nch w=1u l=180n
M1336 t334 nw333 0 0 nch w=1u l=180n
Cnw334 nw334 0 2f
M1337 nw335 nr4 vdd vdd pch w=2u l=180n
M1338 nw335 nw333 vdd vdd pch w=2u l=180n
CT335 t335 0 0.1f
M1339 nw335 nr4 t335 0 nch w=1u l=180n
M1340 t335 nw333 0 0 nch w=1u l=180n
Cnw335 nw335 0 2f
M1341 nw336 nw334 vdd vdd pch w=2u l=180n
M1342 nw336 nw335 vdd vdd pch w=2u l=180n
CT336 t336 0 0.1f
M1343 nw336 nw334 t336 0 nch w=1u l=180n
M1344 t336 nw335 0 0 nch w=1u l=180n
Cnw336 nw336 0 2f
M1345 nw337 nd26 vdd vdd pch w=2u l=180n
M1346 nw337 nd27 vdd vdd pch w=2u l=180n
CT337 t337 0 0.1f
M1347 nw337 nd26 t337 0 nch w=1u l=180n
M1348 t337 nd27 0 0 nch w=1u l=180n
Cnw337 nw337 0 2f
M1349 nw338 nd26 vdd vdd pch w=2u l=180n
M1350 nw338 nw337 vdd vdd pch w=2u l=180n
CT338 t338 0 0.1f
M1351 nw338 nd26 t338 0 nch w=1u l=180n
M1352 t338 nw337 0 0 nch w=1u l=180n
Cnw338 nw338 0 2f
M1353 nw339 nd27 vdd vdd pch w=2u l=180n
M1354 nw339 nw337 vdd vdd pch w=2u l=180n
CT339 t339 0 0.1f
M1355 nw339 nd27 t339 0 nch w=1u l=180n
M1356 t339 nw337 0 0 nch w=1u l=180n
Cnw339 nw339 0 2f
M1357 nw340 nw338 vdd vdd pch w=2u l=180n
M1358 nw340 nw339 vdd vdd pch w=2u l=180n
CT340 t340 0 0.1f
M1359 nw340 nw338 t340 0 nch w=1u l=180n
M1360 t340 nw339 0 0 nch w=1u l=180n
Cnw340 nw340 0 2f
M1361 nw341 nw340 vdd vdd pch w=2u l=180n
M1362 nw341 nd28 vdd vdd pch w=2u l=180n
CT341 t341 0 0.1f
M1363 nw341 nw340 t341 0 nch w=1u l=180n
M1364 t341 nd28 0 0 nch w=1u l=180n
Cnw341 nw341 0 2f
M1365 nw342 nw340 vdd vdd pch w=2u l=180n
M1366 nw342 nw341 vdd vdd pch w=2u l=180n
CT342 t342 0 0.1f
M1367 nw342 nw340 t342 0 nch w=1u l=180n
M1368 t342 nw341 0 0 nch w=1u l=180n
Cnw342 nw342 0 2f
M1369 nw343 nd28 vdd vdd pch w=2u l=180n
M1370 nw343 nw341 vdd vdd pch w=2u l=180n
CT343 t343 0 0.1f
M1371 nw343 nd28 t343 0 nch w=1u l=180n
M1372 t343 nw341 0 0 nch w=1u l=180n
Cnw343 nw343 0 2f
M1373 nw344 nw342 vdd vdd pch w=2u l=180n
M1374 nw344 nw343 vdd vdd pch w=2u l=180n
CT344 t344 0 0.1f
M1375 nw344 nw342 t344 0 nch w=1u l=180n
M1376 t344 nw343 0 0 nch w=1u l=180n
Cnw344 nw344 0 2f
M1377 nw345 nw344 vdd vdd pch w=2u l=180n
M1378 nw345 nd29 vdd vdd pch w=2u l=180n
CT345 t345 0 0.1f
M1379 nw345 nw344 t345 0 nch w=1u l=180n
M1380 t345 nd29 0 0 nch w=1u l=180n
Cnw345 nw345 0 2f
M1381 nw346 nw344 vdd vdd pch w=2u l=180n
M1382 nw346 nw345 vdd vdd pch w=2u l=180n
CT346 t346 0 0.1f
M1383 nw346 nw344 t346 0 nch w=1u l=180n
M1384 t346 nw345 0 0 nch w=1u l=180n
Cnw346 nw346 0 2f
M1385 nw347 nd29 vdd vdd pch w=2u l=180n
M1386 nw347 nw345 vdd vdd pch w=2u l=180n
CT347 t347 0 0.1f
M1387 nw347 nd29 t347 0 nch w=1u l=180n
M1388 t347 nw345 0 0 nch w=1u l=180n
Cnw347 nw347 0 2f
M1389 nw348 nw346 vdd vdd pch w=2u l=180n
M1390 nw348 nw347 vdd vdd pch w=2u l=180n
CT348 t348 0 0.1f
M1391 nw348 nw346 t348 0 nch w=1u l=180n
M1392 t348 nw347 0 0 nch w=1u l=180n
Cnw348 nw348 0 2f
M1393 nw349 nw348 vdd vdd pch w=2u l=180n
M1394 nw349 nd30 vdd vdd pch w=2u l=180n
CT349 t349 0 0.1f
M1395 nw349 nw348 t349 0 nch w=1u l=180n
M1396 t349 nd30 0 0 nch w=1u l=180n
Cnw349 nw349 0 2f
M1397 nw350 nw348 vdd vdd pch w=2u l=180n
M1398 nw350 nw349 vdd vdd pch w=2u l=180n
CT350 t350 0 0.1f
M1399 nw350 nw348 t350 0 nch w=1u l=180n
M1400 t350 nw349 0 0 nch w=1u l=180n
Cnw350 nw350 0 2f
M1401 nw351 nd30 vdd vdd pch w=2u l=180n
M1402 nw351 nw349 vdd vdd pch w=2u l=180n
CT351 t351 0 0.1f
M1403 nw351 nd30 t351 0 nch w=1u l=180n
M1404 t351 nw349 0 0 nch w=1u l=180n
Cnw351 nw351 0 2f
M1405 nw352 nw350 vdd vdd pch w=2u l=180n
M1406 nw352 nw351 vdd vdd pch w=2u l=180n
CT352 t352 0 0.1f
M1407 nw352 nw350 t352 0 nch w=1u l=180n
M1408 t352 nw351 0 0 nch w=1u l=180n
Cnw352 nw352 0 2f
M1409 nw353 nw352 vdd vdd pch w=2u l=180n
M1410 nw353 nd31 vdd vdd pch w=2u l=180n
CT353 t353 0 0.1f
M1411 nw353 nw352 t353 0 nch w=1u l=180n
M1412 t353 nd31 0 0 nch w=1u l=180n
Cnw353 nw353 0 2f
M1413 nw354 nw352 vdd vdd pch w=2u l=180n
M1414 nw354 nw353 vdd vdd pch w=2u l=180n
CT354 t354 0 0.1f
M1415 nw354 nw352 t354 0 nch w=1u l=180n
M1416 t354 nw353 0 0 nch w=1u l=180n
Cnw354 nw354 0 2f
M1417 nw355 nd31 vdd vdd pch w=2u l=180n
M1418 nw355 nw353 vdd vdd pch w=2u l=180n
CT355 t355 0 0.1f
M1419 nw355 nd31 t355 0 nch w=1u l=180n
M1420 t355 nw353 0 0 nch w=1u l=180n
Cnw355 nw355 0 2f
M1421 nw356 nw354 vdd vdd pch w=2u l=180n
M1422 nw356 nw355 vdd vdd pch w=2u l=180n
CT356 t356 0 0.1f
M1423 nw356 nw354 t356 0 nch w=1u l=180n
M1424 t356 nw355 0 0 nch w=1u l=180n
Cnw356 nw356 0 2f
M1425 nw357 nw356 vdd vdd pch w=2u l=180n
M1426 nw357 nr5 vdd vdd pch w=2u l=180n
CT357 t357 0 0.1f
M1427 nw357 nw356 t357 0 nch w=1u l=180n
M1428 t357 nr5 0 0 nch w=1u l=180n
Cnw357 nw357 0 2f
M1429 nw358 nw356 vdd vdd pch w=2u l=180n
M1430 nw358 nw357 vdd vdd pch w=2u l=180n
CT358 t358 0 0.1f
M1431 nw358 nw356 t358 0 nch w=1u l=180n
M1432 t358 nw357 0 0 nch w=1u l=180n
Cnw358 nw358 0 2f
M1433 nw359 nr5 vdd vdd pch w=2u l=180n
M1434 nw359 nw357 vdd vdd pch w=2u l=180n
CT359 t359 0 0.1f
M1435 nw359 nr5 t359 0 nch w=1u l=180n
M1436 t359 nw357 0 0 nch w=1u l=180n
Cnw359 nw359 0 2f
M1437 nw360 nw358 vdd vdd pch w=2u l=180n
M1438 nw360 nw359 vdd vdd pch w=2u l=180n
CT360 t360 0 0.1f
M1439 nw360 nw358 t360 0 nch w=1u l=180n
M1440 t360 nw359 0 0 nch w=1u l=180n
Cnw360 nw360 0 2f
M1441 nw361 nw72 vdd vdd pch w=2u l=180n
M1442 nw361 nw72 0 0 nch w=1u l=180n
Cnw361 nw361 0 2f
M1443 nw362 nw144 vdd vdd pch w=2u l=180n
M1444 nw362 nw144 0 0 nch w=1u l=180n
Cnw362 nw362 0 2f
M1445 nw363 nw216 vdd vdd pch w=2u l=180n
M1446 nw363 nw216 0 0 nch w=1u l=180n
Cnw363 nw363 0 2f
M1447 nw364 nw276 vdd vdd pch w=2u l=180n
M1448 nw364 nw276 0 0 nch w=1u l=180n
Cnw364 nw364 0 2f
M1449 nw365 nw336 vdd vdd pch w=2u l=180n
M1450 nw365 nw336 0 0 nch w=1u l=180n
Cnw365 nw365 0 2f
M1451 nw366 nw360 vdd vdd pch w=2u l=180n
M1452 nw366 nw360 0 0 nch w=1u l=180n
Cnw366 nw366 0 2f
CT361 t361 0 0.1f
M1453 t361 nw72 vdd vdd pch w=2u l=180n
M1454 t361 nw144 vdd vdd pch w=2u l=180n
M1455 t361 nw363 vdd vdd pch w=2u l=180n
M1456 t361 nw364 vdd vdd pch w=2u l=180n
M1457 t361 nw365 vdd vdd pch w=2u l=180n
M1458 t361 nw366 vdd vdd pch w=2u l=180n
M1459 t361 nen vdd vdd pch w=2u l=180n
CT362 t362 0 0.1f
M1460 t361 nw72 t362 0 nch w=1u l=180n
CT363 t363 0 0.1f
M1461 t362 nw144 t363 0 nch w=1u l=180n
CT364 t364 0 0.1f
M1462 t363 nw363 t364 0 nch w=1u l=180n
CT365 t365 0 0.1f
M1463 t364 nw364 t365 0 nch w=1u l=180n
CT366 t366 0 0.1f
M1464 t365 nw365 t366 0 nch w=1u l=180n
CT367 t367 0 0.1f
M1465 t366 nw366 t367 0 nch w=1u l=180n
M1466 t367 nen 0 0 nch w=1u l=180n
M1467 nw367 t361 vdd vdd pch w=2u l=180n
M1468 nw367 t361 0 0 nch w=1u l=180n
Cnw367 nw367 0 2f
M1469 nw368 nd0 vdd vdd pch w=2u l=180n
M1470 nw368 nw367 vdd vdd pch w=2u l=180n
CT368 t368 0 0.1f
M1471 nw368 nd0 t368 0 nch w=1u l=180n
M1472 t368 nw367 0 0 nch w=1u l=180n
Cnw368 nw368 0 2f
M1473 nw369 nd0 vdd vdd pch w=2u l=180n
M1474 nw369 nw368 vdd vdd pch w=2u l=180n
CT369 t369 0 0.1f
M1475 nw369 nd0 t369 0 nch w=1u l=180n
M1476 t369 nw368 0 0 nch w=1u l=180n
Cnw369 nw369 0 2f
M1477 nw370 nw367 vdd vdd pch w=2u l=180n
M1478 nw370 nw368 vdd vdd pch w=2u l=180n
CT370 t370 0 0.1f
M1479 nw370 nw367 t370 0 nch w=1u l=180n
M1480 t370 nw368 0 0 nch w=1u l=180n
Cnw370 nw370 0 2f
M1481 nw371 nw369 vdd vdd pch w=2u l=180n
M1482 nw371 nw370 vdd vdd pch w=2u l=180n
CT371 t371 0 0.1f
M1483 nw371 nw369 t371 0 nch w=1u l=180n
M1484 t371 nw370 0 0 nch w=1u l=180n
Cnw371 nw371 0 2f
CT372 t372 0 0.1f
M1485 t372 nw371 vdd vdd pch w=2u l=180n
M1486 t372 nw371 0 0 nch w=1u l=180n
M1487 nq0 t372 vdd vdd pch w=2u l=180n
M1488 nq0 t372 0 0 nch w=1u l=180n
Cnq0 nq0 0 2f
CT373 t373 0 0.1f
M1489 t373 nw72 vdd vdd pch w=2u l=180n
M1490 t373 nw362 vdd vdd pch w=2u l=180n
M1491 t373 nw216 vdd vdd pch w=2u l=180n
M1492 t373 nw364 vdd vdd pch w=2u l=180n
M1493 t373 nw365 vdd vdd pch w=2u l=180n
M1494 t373 nw366 vdd vdd pch w=2u l=180n
M1495 t373 nen vdd vdd pch w=2u l=180n
CT374 t374 0 0.1f
M1496 t373 nw72 t374 0 nch w=1u l=180n
CT375 t375 0 0.1f
M1497 t374 nw362 t375 0 nch w=1u l=180n
CT376 t376 0 0.1f
M1498 t375 nw216 t376 0 nch w=1u l=180n
CT377 t377 0 0.1f
M1499 t376 nw364 t377 0 nch w=1u l=180n
CT378 t378 0 0.1f
M1500 t377 nw365 t378 0 nch w=1u l=180n
CT379 t379 0 0.1f
M1501 t378 nw366 t379 0 nch w=1u l=180n
M1502 t379 nen 0 0 nch w=1u l=180n
M1503 nw373 t373 vdd vdd pch w=2u l=180n
M1504 nw373 t373 0 0 nch w=1u l=180n
Cnw373 nw373 0 2f
M1505 nw374 nd1 vdd vdd pch w=2u l=180n
M1506 nw374 nw373 vdd vdd pch w=2u l=180n
CT380 t380 0 0.1f
M1507 nw374 nd1 t380 0 nch w=1u l=180n
M1508 t380 nw373 0 0 nch w=1u l=180n
Cnw374 nw374 0 2f
M1509 nw375 nd1 vdd vdd pch w=2u l=180n
M1510 nw375 nw374 vdd vdd pch w=2u l=180n
CT381 t381 0 0.1f
M1511 nw375 nd1 t381 0 nch w=1u l=180n
M1512 t381 nw374 0 0 nch w=1u l=180n
Cnw375 nw375 0 2f
M1513 nw376 nw373 vdd vdd pch w=2u l=180n
M1514 nw376 nw374 vdd vdd pch w=2u l=180n
CT382 t382 0 0.1f
M1515 nw376 nw373 t382 0 nch w=1u l=180n
M1516 t382 nw374 0 0 nch w=1u l=180n
Cnw376 nw376 0 2f
M1517 nw377 nw375 vdd vdd pch w=2u l=180n
M1518 nw377 nw376 vdd vdd pch w=2u l=180n
CT383 t383 0 0.1f
M1519 nw377 nw375 t383 0 nch w=1u l=180n
M1520 t383 nw376 0 0 nch w=1u l=180n
Cnw377 nw377 0 2f
CT384 t384 0 0.1f
M1521 t384 nw377 vdd vdd pch w=2u l=180n
M1522 t384 nw377 0 0 nch w=1u l=180n
M1523 nq1 t384 vdd vdd pch w=2u l=180n
M1524 nq1 t384 0 0 nch w=1u l=180n
Cnq1 nq1 0 2f
CT385 t385 0 0.1f
M1525 t385 nw361 vdd vdd pch w=2u l=180n
M1526 t385 nw144 vdd vdd pch w=2u l=180n
M1527 t385 nw216 vdd vdd pch w=2u l=180n
M1528 t385 nw364 vdd vdd pch w=2u l=180n
M1529 t385 nw365 vdd vdd pch w=2u l=180n
M1530 t385 nw366 vdd vdd pch w=2u l=180n
M1531 t385 nen vdd vdd pch w=2u l=180n
CT386 t386 0 0.1f
M1532 t385 nw361 t386 0 nch w=1u l=180n
CT387 t387 0 0.1f
M1533 t386 nw144 t387 0 nch w=1u l=180n
CT388 t388 0 0.1f
M1534 t387 nw216 t388 0 nch w=1u l=180n
CT389 t389 0 0.1f
M1535 t388 nw364 t389 0 nch w=1u l=180n
CT390 t390 0 0.1f
M1536 t389 nw365 t390 0 nch w=1u l=180n
CT391 t391 0 0.1f
M1537 t390 nw366 t391 0 nch w=1u l=180n
M1538 t391 nen 0 0 nch w=1u l=180n
M1539 nw379 t385 vdd vdd pch w=2u l=180n
M1540 nw379 t385 0 0 nch w=1u l=180n
Cnw379 nw379 0 2f
M1541 nw380 nd2 vdd vdd pch w=2u l=180n
M1542 nw380 nw379 vdd vdd pch w=2u l=180n
CT392 t392 0 0.1f
M1543 nw380 nd2 t392 0 nch w=1u l=180n
M1544 t392 nw379 0 0 nch w=1u l=180n
Cnw380 nw380 0 2f
M1545 nw381 nd2 vdd vdd pch w=2u l=180n
M1546 nw381 nw380 vdd vdd pch w=2u l=180n
CT393 t393 0 0.1f
M1547 nw381 nd2 t393 0 nch w=1u l=180n
M1548 t393 nw380 0 0 nch w=1u l=180n
Cnw381 nw381 0 2f
M1549 nw382 nw379 vdd vdd pch w=2u l=180n
M1550 nw382 nw380 vdd vdd pch w=2u l=180n
CT394 t394 0 0.1f
M1551 nw382 nw379 t394 0 nch w=1u l=180n
M1552 t394 nw380 0 0 nch w=1u l=180n
Cnw382 nw382 0 2f
M1553 nw383 nw381 vdd vdd pch w=2u l=180n
M1554 nw383 nw382 vdd vdd pch w=2u l=180n
CT395 t395 0 0.1f
M1555 nw383 nw381 t395 0 nch w=1u l=180n
M1556 t395 nw382 0 0 nch w=1u l=180n
Cnw383 nw383 0 2f
CT396 t396 0 0.1f
M1557 t396 nw383 vdd vdd pch w=2u l=180n
M1558 t396 nw383 0 0 nch w=1u l=180n
M1559 nq2 t396 vdd vdd pch w=2u l=180n
M1560 nq2 t396 0 0 nch w=1u l=180n
Cnq2 nq2 0 2f
CT397 t397 0 0.1f
M1561 t397 nw72 vdd vdd pch w=2u l=180n
M1562 t397 nw144 vdd vdd pch w=2u l=180n
M1563 t397 nw216 vdd vdd pch w=2u l=180n
M1564 t397 nw364 vdd vdd pch w=2u l=180n
M1565 t397 nw365 vdd vdd pch w=2u l=180n
M1566 t397 nw366 vdd vdd pch w=2u l=180n
M1567 t397 nen vdd vdd pch w=2u l=180n
CT398 t398 0 0.1f
M1568 t397 nw72 t398 0 nch w=1u l=180n
CT399 t399 0 0.1f
M1569 t398 nw144 t399 0 nch w=1u l=180n
CT400 t400 0 0.1f
M1570 t399 nw216 t400 0 nch w=1u l=180n
CT401 t401 0 0.1f
M1571 t400 nw364 t401 0 nch w=1u l=180n
CT402 t402 0 0.1f
M1572 t401 nw365 t402 0 nch w=1u l=180n
CT403 t403 0 0.1f
M1573 t402 nw366 t403 0 nch w=1u l=180n
M1574 t403 nen 0 0 nch w=1u l=180n
M1575 nw385 t397 vdd vdd pch w=2u l=180n
M1576 nw385 t397 0 0 nch w=1u l=180n
Cnw385 nw385 0 2f
M1577 nw386 nd3 vdd vdd pch w=2u l=180n
M1578 nw386 nw385 vdd vdd pch w=2u l=180n
CT404 t404 0 0.1f
M1579 nw386 nd3 t404 0 nch w=1u l=180n
M1580 t404 nw385 0 0 nch w=1u l=180n
Cnw386 nw386 0 2f
M1581 nw387 nd3 vdd vdd pch w=2u l=180n
M1582 nw387 nw386 vdd vdd pch w=2u l=180n
CT405 t405 0 0.1f
M1583 nw387 nd3 t405 0 nch w=1u l=180n
M1584 t405 nw386 0 0 nch w=1u l=180n
Cnw387 nw387 0 2f
M1585 nw388 nw385 vdd vdd pch w=2u l=180n
M1586 nw388 nw386 vdd vdd pch w=2u l=180n
CT406 t406 0 0.1f
M1587 nw388 nw385 t406 0 nch w=1u l=180n
M1588 t406 nw386 0 0 nch w=1u l=180n
Cnw388 nw388 0 2f
M1589 nw389 nw387 vdd vdd pch w=2u l=180n
M1590 nw389 nw388 vdd vdd pch w=2u l=180n
CT407 t407 0 0.1f
M1591 nw389 nw387 t407 0 nch w=1u l=180n
M1592 t407 nw388 0 0 nch w=1u l=180n
Cnw389 nw389 0 2f
CT408 t408 0 0.1f
M1593 t408 nw389 vdd vdd pch w=2u l=180n
M1594 t408 nw389 0 0 nch w=1u l=180n
M1595 nq3 t408 vdd vdd pch w=2u l=180n
M1596 nq3 t408 0 0 nch w=1u l=180n
Cnq3 nq3 0 2f
CT409 t409 0 0.1f
M1597 t409 nw72 vdd vdd pch w=2u l=180n
M1598 t409 nw362 vdd vdd pch w=2u l=180n
M1599 t409 nw363 vdd vdd pch w=2u l=180n
M1600 t409 nw276 vdd vdd pch w=2u l=180n
M1601 t409 nw365 vdd vdd pch w=2u l=180n
M1602 t409 nw366 vdd vdd pch w=2u l=180n
M1603 t409 nen vdd vdd pch w=2u l=180n
CT410 t410 0 0.1f
M1604 t409 nw72 t410 0 nch w=1u l=180n
CT411 t411 0 0.1f
M1605 t410 nw362 t411 0 nch w=1u l=180n
CT412 t412 0 0.1f
M1606 t411 nw363 t412 0 nch w=1u l=180n
CT413 t413 0 0.1f
M1607 t412 nw276 t413 0 nch w=1u l=180n
CT414 t414 0 0.1f
M1608 t413 nw365 t414 0 nch w=1u l=180n
CT415 t415 0 0.1f
M1609 t414 nw366 t415 0 nch w=1u l=180n
M1610 t415 nen 0 0 nch w=1u l=180n
M1611 nw391 t409 vdd vdd pch w=2u l=180n
M1612 nw391 t409 0 0 nch w=1u l=180n
Cnw391 nw391 0 2f
M1613 nw392 nd4 vdd vdd pch w=2u l=180n
M1614 nw392 nw391 vdd vdd pch w=2u l=180n
CT416 t416 0 0.1f
M1615 nw392 nd4 t416 0 nch w=1u l=180n
M1616 t416 nw391 0 0 nch w=1u l=180n
Cnw392 nw392 0 2f
M1617 nw393 nd4 vdd vdd pch w=2u l=180n
M1618 nw393 nw392 vdd vdd pch w=2u l=180n
CT417 t417 0 0.1f
M1619 nw393 nd4 t417 0 nch w=1u l=180n
M1620 t417 nw392 0 0 nch w=1u l=180n
Cnw393 nw393 0 2f
M1621 nw394 nw391 vdd vdd pch w=2u l=180n
M1622 nw394 nw392 vdd vdd pch w=2u l=180n
CT418 t418 0 0.1f
M1623 nw394 nw391 t418 0 nch w=1u l=180n
M1624 t418 nw392 0 0 nch w=1u l=180n
Cnw394 nw394 0 2f
M1625 nw395 nw393 vdd vdd pch w=2u l=180n
M1626 nw395 nw394 vdd vdd pch w=2u l=180n
CT419 t419 0 0.1f
M1627 nw395 nw393 t419 0 nch w=1u l=180n
M1628 t419 nw394 0 0 nch w=1u l=180n
Cnw395 nw395 0 2f
CT420 t420 0 0.1f
M1629 t420 nw395 vdd vdd pch w=2u l=180n
M1630 t420 nw395 0 0 nch w=1u l=180n
M1631 nq4 t420 vdd vdd pch w=2u l=180n
M1632 nq4 t420 0 0 nch w=1u l=180n
Cnq4 nq4 0 2f
CT421 t421 0 0.1f
M1633 t421 nw361 vdd vdd pch w=2u l=180n
M1634 t421 nw144 vdd vdd pch w=2u l=180n
M1635 t421 nw363 vdd vdd pch w=2u l=180n
M1636 t421 nw276 vdd vdd pch w=2u l=180n
M1637 t421 nw365 vdd vdd pch w=2u l=180n
M1638 t421 nw366 vdd vdd pch w=2u l=180n
M1639 t421 nen vdd vdd pch w=2u l=180n
CT422 t422 0 0.1f
M1640 t421 nw361 t422 0 nch w=1u l=180n
CT423 t423 0 0.1f
M1641 t422 nw144 t423 0 nch w=1u l=180n
CT424 t424 0 0.1f
M1642 t423 nw363 t424 0 nch w=1u l=180n
CT425 t425 0 0.1f
M1643 t424 nw276 t425 0 nch w=1u l=180n
CT426 t426 0 0.1f
M1644 t425 nw365 t426 0 nch w=1u l=180n
CT427 t427 0 0.1f
M1645 t426 nw366 t427 0 nch w=1u l=180n
M1646 t427 nen 0 0 nch w=1u l=180n
M1647 nw397 t421 vdd vdd pch w=2u l=180n
M1648 nw397 t421 0 0 nch w=1u l=180n
Cnw397 nw397 0 2f
M1649 nw398 nd5 vdd vdd pch w=2u l=180n
M1650 nw398 nw397 vdd vdd pch w=2u l=180n
CT428 t428 0 0.1f
M1651 nw398 nd5 t428 0 nch w=1u l=180n
M1652 t428 nw397 0 0 nch w=1u l=180n
Cnw398 nw398 0 2f
M1653 nw399 nd5 vdd vdd pch w=2u l=180n
M1654 nw399 nw398 vdd vdd pch w=2u l=180n
CT429 t429 0 0.1f
M1655 nw399 nd5 t429 0 nch w=1u l=180n
M1656 t429 nw398 0 0 nch w=1u l=180n
Cnw399 nw399 0 2f
M1657 nw400 nw397 vdd vdd pch w=2u l=180n
M1658 nw400 nw398 vdd vdd pch w=2u l=180n
CT430 t430 0 0.1f
M1659 nw400 nw397 t430 0 nch w=1u l=180n
M1660 t430 nw398 0 0 nch w=1u l=180n
Cnw400 nw400 0 2f
M1661 nw401 nw399 vdd vdd pch w=2u l=180n
M1662 nw401 nw400 vdd vdd pch w=2u l=180n
CT431 t431 0 0.1f
M1663 nw401 nw399 t431 0 nch w=1u l=180n
M1664 t431 nw400 0 0 nch w=1u l=180n
Cnw401 nw401 0 2f
CT432 t432 0 0.1f
M1665 t432 nw401 vdd vdd pch w=2u l=180n
M1666 t432 nw401 0 0 nch w=1u l=180n
M1667 nq5 t432 vdd vdd pch w=2u l=180n
M1668 nq5 t432 0 0 nch w=1u l=180n
Cnq5 nq5 0 2f
CT433 t433 0 0.1f
M1669 t433 nw72 vdd vdd pch w=2u l=180n
M1670 t433 nw144 vdd vdd pch w=2u l=180n
M1671 t433 nw363 vdd vdd pch w=2u l=180n
M1672 t433 nw276 vdd vdd pch w=2u l=180n
M1673 t433 nw365 vdd vdd pch w=2u l=180n
M1674 t433 nw366 vdd vdd pch w=2u l=180n
M1675 t433 nen vdd vdd pch w=2u l=180n
CT434 t434 0 0.1f
M1676 t433 nw72 t434 0 nch w=1u l=180n
CT435 t435 0 0.1f
M1677 t434 nw144 t435 0 nch w=1u l=180n
CT436 t436 0 0.1f
M1678 t435 nw363 t436 0 nch w=1u l=180n
CT437 t437 0 0.1f
M1679 t436 nw276 t437 0 nch w=1u l=180n
CT438 t438 0 0.1f
M1680 t437 nw365 t438 0 nch w=1u l=180n
CT439 t439 0 0.1f
M1681 t438 nw366 t439 0 nch w=1u l=180n
M1682 t439 nen 0 0 nch w=1u l=180n
M1683 nw403 t433 vdd vdd pch w=2u l=180n
M1684 nw403 t433 0 0 nch w=1u l=180n
Cnw403 nw403 0 2f
M1685 nw404 nd6 vdd vdd pch w=2u l=180n
M1686 nw404 nw403 vdd vdd pch w=2u l=180n
CT440 t440 0 0.1f
M1687 nw404 nd6 t440 0 nch w=1u l=180n
M1688 t440 nw403 0 0 nch w=1u l=180n
Cnw404 nw404 0 2f
M1689 nw405 nd6 vdd vdd pch w=2u l=180n
M1690 nw405 nw404 vdd vdd pch w=2u l=180n
CT441 t441 0 0.1f
M1691 nw405 nd6 t441 0 nch w=1u l=180n
M1692 t441 nw404 0 0 nch w=1u l=180n
Cnw405 nw405 0 2f
M1693 nw406 nw403 vdd vdd pch w=2u l=180n
M1694 nw406 nw404 vdd vdd pch w=2u l=180n
CT442 t442 0 0.1f
M1695 nw406 nw403 t442 0 nch w=1u l=180n
M1696 t442 nw404 0 0 nch w=1u l=180n
Cnw406 nw406 0 2f
M1697 nw407 nw405 vdd vdd pch w=2u l=180n
M1698 nw407 nw406 vdd vdd pch w=2u l=180n
CT443 t443 0 0.1f
M1699 nw407 nw405 t443 0 nch w=1u l=180n
M1700 t443 nw406 0 0 nch w=1u l=180n
Cnw407 nw407 0 2f
CT444 t444 0 0.1f
M1701 t444 nw407 vdd vdd pch w=2u l=180n
M1702 t444 nw407 0 0 nch w=1u l=180n
M1703 nq6 t444 vdd vdd pch w=2u l=180n
M1704 nq6 t444 0 0 nch w=1u l=180n
Cnq6 nq6 0 2f
CT445 t445 0 0.1f
M1705 t445 nw361 vdd vdd pch w=2u l=180n
M1706 t445 nw362 vdd vdd pch w=2u l=180n
M1707 t445 nw216 vdd vdd pch w=2u l=180n
M1708 t445 nw276 vdd vdd pch w=2u l=180n
M1709 t445 nw365 vdd vdd pch w=2u l=180n
M1710 t445 nw366 vdd vdd pch w=2u l=180n
M1711 t445 nen vdd vdd pch w=2u l=180n
CT446 t446 0 0.1f
M1712 t445 nw361 t446 0 nch w=1u l=180n
CT447 t447 0 0.1f
M1713 t446 nw362 t447 0 nch w=1u l=180n
CT448 t448 0 0.1f
M1714 t447 nw216 t448 0 nch w=1u l=180n
CT449 t449 0 0.1f
M1715 t448 nw276 t449 0 nch w=1u l=180n
CT450 t450 0 0.1f
M1716 t449 nw365 t450 0 nch w=1u l=180n
CT451 t451 0 0.1f
M1717 t450 nw366 t451 0 nch w=1u l=180n
M1718 t451 nen 0 0 nch w=1u l=180n
M1719 nw409 t445 vdd vdd pch w=2u l=180n
M1720 nw409 t445 0 0 nch w=1u l=180n
Cnw409 nw409 0 2f
M1721 nw410 nd7 vdd vdd pch w=2u l=180n
M1722 nw410 nw409 vdd vdd pch w=2u l=180n
CT452 t452 0 0.1f
M1723 nw410 nd7 t452 0 nch w=1u l=180n
M1724 t452 nw409 0 0 nch w=1u l=180n
Cnw410 nw410 0 2f
M1725 nw411 nd7 vdd vdd pch w=2u l=180n
M1726 nw411 nw410 vdd vdd pch w=2u l=180n
CT453 t453 0 0.1f
M1727 nw411 nd7 t453 0 nch w=1u l=180n
M1728 t453 nw410 0 0 nch w=1u l=180n
Cnw411 nw411 0 2f
M1729 nw412 nw409 vdd vdd pch w=2u l=180n
M1730 nw412 nw410 vdd vdd pch w=2u l=180n
CT454 t454 0 0.1f
M1731 nw412 nw409 t454 0 nch w=1u l=180n
M1732 t454 nw410 0 0 nch w=1u l=180n
Cnw412 nw412 0 2f
M1733 nw413 nw411 vdd vdd pch w=2u l=180n
M1734 nw413 nw412 vdd vdd pch w=2u l=180n
CT455 t455 0 0.1f
M1735 nw413 nw411 t455 0 nch w=1u l=180n
M1736 t455 nw412 0 0 nch w=1u l=180n
Cnw413 nw413 0 2f
CT456 t456 0 0.1f
M1737 t456 nw413 vdd vdd pch w=2u l=180n
M1738 t456 nw413 0 0 nch w=1u l=180n
M1739 nq7 t456 vdd vdd pch w=2u l=180n
M1740 nq7 t456 0 0 nch w=1u l=180n
Cnq7 nq7 0 2f
CT457 t457 0 0.1f
M1741 t457 nw72 vdd vdd pch w=2u l=180n
M1742 t457 nw362 vdd vdd pch w=2u l=180n
M1743 t457 nw216 vdd vdd pch w=2u l=180n
M1744 t457 nw276 vdd vdd pch w=2u l=180n
M1745 t457 nw365 vdd vdd pch w=2u l=180n
M1746 t457 nw366 vdd vdd pch w=2u l=180n
M1747 t457 nen vdd vdd pch w=2u l=180n
CT458 t458 0 0.1f
M1748 t457 nw72 t458 0 nch w=1u l=180n
CT459 t459 0 0.1f
M1749 t458 nw362 t459 0 nch w=1u l=180n
CT460 t460 0 0.1f
M1750 t459 nw216 t460 0 nch w=1u l=180n
CT461 t461 0 0.1f
M1751 t460 nw276 t461 0 nch w=1u l=180n
CT462 t462 0 0.1f
M1752 t461 nw365 t462 0 nch w=1u l=180n
CT463 t463 0 0.1f
M1753 t462 nw366 t463 0 nch w=1u l=180n
M1754 t463 nen 0 0 nch w=1u l=180n
M1755 nw415 t457 vdd vdd pch w=2u l=180n
M1756 nw415 t457 0 0 nch w=1u l=180n
Cnw415 nw415 0 2f
M1757 nw416 nd8 vdd vdd pch w=2u l=180n
M1758 nw416 nw415 vdd vdd pch w=2u l=180n
CT464 t464 0 0.1f
M1759 nw416 nd8 t464 0 nch w=1u l=180n
M1760 t464 nw415 0 0 nch w=1u l=180n
Cnw416 nw416 0 2f
M1761 nw417 nd8 vdd vdd pch w=2u l=180n
M1762 nw417 nw416 vdd vdd pch w=2u l=180n
CT465 t465 0 0.1f
M1763 nw417 nd8 t465 0 nch w=1u l=180n
M1764 t465 nw416 0 0 nch w=1u l=180n
Cnw417 nw417 0 2f
M1765 nw418 nw415 vdd vdd pch w=2u l=180n
M1766 nw418 nw416 vdd vdd pch w=2u l=180n
CT466 t466 0 0.1f
M1767 nw418 nw415 t466 0 nch w=1u l=180n
M1768 t466 nw416 0 0 nch w=1u l=180n
Cnw418 nw418 0 2f
M1769 nw419 nw417 vdd vdd pch w=2u l=180n
M1770 nw419 nw418 vdd vdd pch w=2u l=180n
CT467 t467 0 0.1f
M1771 nw419 nw417 t467 0 nch w=1u l=180n
M1772 t467 nw418 0 0 nch w=1u l=180n
Cnw419 nw419 0 2f
CT468 t468 0 0.1f
M1773 t468 nw419 vdd vdd pch w=2u l=180n
M1774 t468 nw419 0 0 nch w=1u l=180n
M1775 nq8 t468 vdd vdd pch w=2u l=180n
M1776 nq8 t468 0 0 nch w=1u l=180n
Cnq8 nq8 0 2f
CT469 t469 0 0.1f
M1777 t469 nw361 vdd vdd pch w=2u l=180n
M1778 t469 nw144 vdd vdd pch w=2u l=180n
M1779 t469 nw216 vdd vdd pch w=2u l=180n
M1780 t469 nw276 vdd vdd pch w=2u l=180n
M1781 t469 nw365 vdd vdd pch w=2u l=180n
M1782 t469 nw366 vdd vdd pch w=2u l=180n
M1783 t469 nen vdd vdd pch w=2u l=180n
CT470 t470 0 0.1f
M1784 t469 nw361 t470 0 nch w=1u l=180n
CT471 t471 0 0.1f
M1785 t470 nw144 t471 0 nch w=1u l=180n
CT472 t472 0 0.1f
M1786 t471 nw216 t472 0 nch w=1u l=180n
CT473 t473 0 0.1f
M1787 t472 nw276 t473 0 nch w=1u l=180n
CT474 t474 0 0.1f
M1788 t473 nw365 t474 0 nch w=1u l=180n
CT475 t475 0 0.1f
M1789 t474 nw366 t475 0 nch w=1u l=180n
M1790 t475 nen 0 0 nch w=1u l=180n
M1791 nw421 t469 vdd vdd pch w=2u l=180n
M1792 nw421 t469 0 0 nch w=1u l=180n
Cnw421 nw421 0 2f
M1793 nw422 nd9 vdd vdd pch w=2u l=180n
M1794 nw422 nw421 vdd vdd pch w=2u l=180n
CT476 t476 0 0.1f
M1795 nw422 nd9 t476 0 nch w=1u l=180n
M1796 t476 nw421 0 0 nch w=1u l=180n
Cnw422 nw422 0 2f
M1797 nw423 nd9 vdd vdd pch w=2u l=180n
M1798 nw423 nw422 vdd vdd pch w=2u l=180n
CT477 t477 0 0.1f
M1799 nw423 nd9 t477 0 nch w=1u l=180n
M1800 t477 nw422 0 0 nch w=1u l=180n
Cnw423 nw423 0 2f
M1801 nw424 nw421 vdd vdd pch w=2u l=180n
M1802 nw424 nw422 vdd vdd pch w=2u l=180n
CT478 t478 0 0.1f
M1803 nw424 nw421 t478 0 nch w=1u l=180n
M1804 t478 nw422 0 0 nch w=1u l=180n
Cnw424 nw424 0 2f
M1805 nw425 nw423 vdd vdd pch w=2u l=180n
M1806 nw425 nw424 vdd vdd pch w=2u l=180n
CT479 t479 0 0.1f
M1807 nw425 nw423 t479 0 nch w=1u l=180n
M1808 t479 nw424 0 0 nch w=1u l=180n
Cnw425 nw425 0 2f
CT480 t480 0 0.1f
M1809 t480 nw425 vdd vdd pch w=2u l=180n
M1810 t480 nw425 0 0 nch w=1u l=180n
M1811 nq9 t480 vdd vdd pch w=2u l=180n
M1812 nq9 t480 0 0 nch w=1u l=180n
Cnq9 nq9 0 2f
CT481 t481 0 0.1f
M1813 t481 nw72 vdd vdd pch w=2u l=180n
M1814 t481 nw144 vdd vdd pch w=2u l=180n
M1815 t481 nw216 vdd vdd pch w=2u l=180n
M1816 t481 nw276 vdd vdd pch w=2u l=180n
M1817 t481 nw365 vdd vdd pch w=2u l=180n
M1818 t481 nw366 vdd vdd pch w=2u l=180n
M1819 t481 nen vdd vdd pch w=2u l=180n
CT482 t482 0 0.1f
M1820 t481 nw72 t482 0 nch w=1u l=180n
CT483 t483 0 0.1f
M1821 t482 nw144 t483 0 nch w=1u l=180n
CT484 t484 0 0.1f
M1822 t483 nw216 t484 0 nch w=1u l=180n
CT485 t485 0 0.1f
M1823 t484 nw276 t485 0 nch w=1u l=180n
CT486 t486 0 0.1f
M1824 t485 nw365 t486 0 nch w=1u l=180n
CT487 t487 0 0.1f
M1825 t486 nw366 t487 0 nch w=1u l=180n
M1826 t487 nen 0 0 nch w=1u l=180n
M1827 nw427 t481 vdd vdd pch w=2u l=180n
M1828 nw427 t481 0 0 nch w=1u l=180n
Cnw427 nw427 0 2f
M1829 nw428 nd10 vdd vdd pch w=2u l=180n
M1830 nw428 nw427 vdd vdd pch w=2u l=180n
CT488 t488 0 0.1f
M1831 nw428 nd10 t488 0 nch w=1u l=180n
M1832 t488 nw427 0 0 nch w=1u l=180n
Cnw428 nw428 0 2f
M1833 nw429 nd10 vdd vdd pch w=2u l=180n
M1834 nw429 nw428 vdd vdd pch w=2u l=180n
CT489 t489 0 0.1f
M1835 nw429 nd10 t489 0 nch w=1u l=180n
M1836 t489 nw428 0 0 nch w=1u l=180n
Cnw429 nw429 0 2f
M1837 nw430 nw427 vdd vdd pch w=2u l=180n
M1838 nw430 nw428 vdd vdd pch w=2u l=180n
CT490 t490 0 0.1f
M1839 nw430 nw427 t490 0 nch w=1u l=180n
M1840 t490 nw428 0 0 nch w=1u l=180n
Cnw430 nw430 0 2f
M1841 nw431 nw429 vdd vdd pch w=2u l=180n
M1842 nw431 nw430 vdd vdd pch w=2u l=180n
CT491 t491 0 0.1f
M1843 nw431 nw429 t491 0 nch w=1u l=180n
M1844 t491 nw430 0 0 nch w=1u l=180n
Cnw431 nw431 0 2f
CT492 t492 0 0.1f
M1845 t492 nw431 vdd vdd pch w=2u l=180n
M1846 t492 nw431 0 0 nch w=1u l=180n
M1847 nq10 t492 vdd vdd pch w=2u l=180n
M1848 nq10 t492 0 0 nch w=1u l=180n
Cnq10 nq10 0 2f
CT493 t493 0 0.1f
M1849 t493 nw72 vdd vdd pch w=2u l=180n
M1850 t493 nw362 vdd vdd pch w=2u l=180n
M1851 t493 nw363 vdd vdd pch w=2u l=180n
M1852 t493 nw364 vdd vdd pch w=2u l=180n
M1853 t493 nw336 vdd vdd pch w=2u l=180n
M1854 t493 nw366 vdd vdd pch w=2u l=180n
M1855 t493 nen vdd vdd pch w=2u l=180n
CT494 t494 0 0.1f
M1856 t493 nw72 t494 0 nch w=1u l=180n
CT495 t495 0 0.1f
M1857 t494 nw362 t495 0 nch w=1u l=180n
CT496 t496 0 0.1f
M1858 t495 nw363 t496 0 nch w=1u l=180n
CT497 t497 0 0.1f
M1859 t496 nw364 t497 0 nch w=1u l=180n
CT498 t498 0 0.1f
M1860 t497 nw336 t498 0 nch w=1u l=180n
CT499 t499 0 0.1f
M1861 t498 nw366 t499 0 nch w=1u l=180n
M1862 t499 nen 0 0 nch w=1u l=180n
M1863 nw433 t493 vdd vdd pch w=2u l=180n
M1864 nw433 t493 0 0 nch w=1u l=180n
Cnw433 nw433 0 2f
M1865 nw434 nd11 vdd vdd pch w=2u l=180n
M1866 nw434 nw433 vdd vdd pch w=2u l=180n
CT500 t500 0 0.1f
M1867 nw434 nd11 t500 0 nch w=1u l=180n
M1868 t500 nw433 0 0 nch w=1u l=180n
Cnw434 nw434 0 2f
M1869 nw435 nd11 vdd vdd pch w=2u l=180n
M1870 nw435 nw434 vdd vdd pch w=2u l=180n
CT501 t501 0 0.1f
M1871 nw435 nd11 t501 0 nch w=1u l=180n
M1872 t501 nw434 0 0 nch w=1u l=180n
Cnw435 nw435 0 2f
M1873 nw436 nw433 vdd vdd pch w=2u l=180n
M1874 nw436 nw434 vdd vdd pch w=2u l=180n
CT502 t502 0 0.1f
M1875 nw436 nw433 t502 0 nch w=1u l=180n
M1876 t502 nw434 0 0 nch w=1u l=180n
Cnw436 nw436 0 2f
M1877 nw437 nw435 vdd vdd pch w=2u l=180n
M1878 nw437 nw436 vdd vdd pch w=2u l=180n
CT503 t503 0 0.1f
M1879 nw437 nw435 t503 0 nch w=1u l=180n
M1880 t503 nw436 0 0 nch w=1u l=180n
Cnw437 nw437 0 2f
CT504 t504 0 0.1f
M1881 t504 nw437 vdd vdd pch w=2u l=180n
M1882 t504 nw437 0 0 nch w=1u l=180n
M1883 nq11 t504 vdd vdd pch w=2u l=180n
M1884 nq11 t504 0 0 nch w=1u l=180n
Cnq11 nq11 0 2f
CT505 t505 0 0.1f
M1885 t505 nw361 vdd vdd pch w=2u l=180n
M1886 t505 nw144 vdd vdd pch w=2u l=180n
M1887 t505 nw363 vdd vdd pch w=2u l=180n
M1888 t505 nw364 vdd vdd pch w=2u l=180n
M1889 t505 nw336 vdd vdd pch w=2u l=180n
M1890 t505 nw366 vdd vdd pch w=2u l=180n
M1891 t505 nen vdd vdd pch w=2u l=180n
CT506 t506 0 0.1f
M1892 t505 nw361 t506 0 nch w=1u l=180n
CT507 t507 0 0.1f
M1893 t506 nw144 t507 0 nch w=1u l=180n
CT508 t508 0 0.1f
M1894 t507 nw363 t508 0 nch w=1u l=180n
CT509 t509 0 0.1f
M1895 t508 nw364 t509 0 nch w=1u l=180n
CT510 t510 0 0.1f
M1896 t509 nw336 t510 0 nch w=1u l=180n
CT511 t511 0 0.1f
M1897 t510 nw366 t511 0 nch w=1u l=180n
M1898 t511 nen 0 0 nch w=1u l=180n
M1899 nw439 t505 vdd vdd pch w=2u l=180n
M1900 nw439 t505 0 0 nch w=1u l=180n
Cnw439 nw439 0 2f
M1901 nw440 nd12 vdd vdd pch w=2u l=180n
M1902 nw440 nw439 vdd vdd pch w=2u l=180n
CT512 t512 0 0.1f
M1903 nw440 nd12 t512 0 nch w=1u l=180n
M1904 t512 nw439 0 0 nch w=1u l=180n
Cnw440 nw440 0 2f
M1905 nw441 nd12 vdd vdd pch w=2u l=180n
M1906 nw441 nw440 vdd vdd pch w=2u l=180n
CT513 t513 0 0.1f
M1907 nw441 nd12 t513 0 nch w=1u l=180n
M1908 t513 nw440 0 0 nch w=1u l=180n
Cnw441 nw441 0 2f
M1909 nw442 nw439 vdd vdd pch w=2u l=180n
M1910 nw442 nw440 vdd vdd pch w=2u l=180n
CT514 t514 0 0.1f
M1911 nw442 nw439 t514 0 nch w=1u l=180n
M1912 t514 nw440 0 0 nch w=1u l=180n
Cnw442 nw442 0 2f
M1913 nw443 nw441 vdd vdd pch w=2u l=180n
M1914 nw443 nw442 vdd vdd pch w=2u l=180n
CT515 t515 0 0.1f
M1915 nw443 nw441 t515 0 nch w=1u l=180n
M1916 t515 nw442 0 0 nch w=1u l=180n
Cnw443 nw443 0 2f
CT516 t516 0 0.1f
M1917 t516 nw443 vdd vdd pch w=2u l=180n
M1918 t516 nw443 0 0 nch w=1u l=180n
M1919 nq12 t516 vdd vdd pch w=2u l=180n
M1920 nq12 t516 0 0 nch w=1u l=180n
Cnq12 nq12 0 2f
CT517 t517 0 0.1f
M1921 t517 nw72 vdd vdd pch w=2u l=180n
M1922 t517 nw144 vdd vdd pch w=2u l=180n
M1923 t517 nw363 vdd vdd pch w=2u l=180n
M1924 t517 nw364 vdd vdd pch w=2u l=180n
M1925 t517 nw336 vdd vdd pch w=2u l=180n
M1926 t517 nw366 vdd vdd pch w=2u l=180n
M1927 t517 nen vdd vdd pch w=2u l=180n
CT518 t518 0 0.1f
M1928 t517 nw72 t518 0 nch w=1u l=180n
CT519 t519 0 0.1f
M1929 t518 nw144 t519 0 nch w=1u l=180n
CT520 t520 0 0.1f
M1930 t519 nw363 t520 0 nch w=1u l=180n
CT521 t521 0 0.1f
M1931 t520 nw364 t521 0 nch w=1u l=180n
CT522 t522 0 0.1f
M1932 t521 nw336 t522 0 nch w=1u l=180n
CT523 t523 0 0.1f
M1933 t522 nw366 t523 0 nch w=1u l=180n
M1934 t523 nen 0 0 nch w=1u l=180n
M1935 nw445 t517 vdd vdd pch w=2u l=180n
M1936 nw445 t517 0 0 nch w=1u l=180n
Cnw445 nw445 0 2f
M1937 nw446 nd13 vdd vdd pch w=2u l=180n
M1938 nw446 nw445 vdd vdd pch w=2u l=180n
CT524 t524 0 0.1f
M1939 nw446 nd13 t524 0 nch w=1u l=180n
M1940 t524 nw445 0 0 nch w=1u l=180n
Cnw446 nw446 0 2f
M1941 nw447 nd13 vdd vdd pch w=2u l=180n
M1942 nw447 nw446 vdd vdd pch w=2u l=180n
CT525 t525 0 0.1f
M1943 nw447 nd13 t525 0 nch w=1u l=180n
M1944 t525 nw446 0 0 nch w=1u l=180n
Cnw447 nw447 0 2f
M1945 nw448 nw445 vdd vdd pch w=2u l=180n
M1946 nw448 nw446 vdd vdd pch w=2u l=180n
CT526 t526 0 0.1f
M1947 nw448 nw445 t526 0 nch w=1u l=180n
M1948 t526 nw446 0 0 nch w=1u l=180n
Cnw448 nw448 0 2f
M1949 nw449 nw447 vdd vdd pch w=2u l=180n
M1950 nw449 nw448 vdd vdd pch w=2u l=180n
CT527 t527 0 0.1f
M1951 nw449 nw447 t527 0 nch w=1u l=180n
M1952 t527 nw448 0 0 nch w=1u l=180n
Cnw449 nw449 0 2f
CT528 t528 0 0.1f
M1953 t528 nw449 vdd vdd pch w=2u l=180n
M1954 t528 nw449 0 0 nch w=1u l=180n
M1955 nq13 t528 vdd vdd pch w=2u l=180n
M1956 nq13 t528 0 0 nch w=1u l=180n
Cnq13 nq13 0 2f
CT529 t529 0 0.1f
M1957 t529 nw361 vdd vdd pch w=2u l=180n
M1958 t529 nw362 vdd vdd pch w=2u l=180n
M1959 t529 nw216 vdd vdd pch w=2u l=180n
M1960 t529 nw364 vdd vdd pch w=2u l=180n
M1961 t529 nw336 vdd vdd pch w=2u l=180n
M1962 t529 nw366 vdd vdd pch w=2u l=180n
M1963 t529 nen vdd vdd pch w=2u l=180n
CT530 t530 0 0.1f
M1964 t529 nw361 t530 0 nch w=1u l=180n
CT531 t531 0 0.1f
M1965 t530 nw362 t531 0 nch w=1u l=180n
CT532 t532 0 0.1f
M1966 t531 nw216 t532 0 nch w=1u l=180n
CT533 t533 0 0.1f
M1967 t532 nw364 t533 0 nch w=1u l=180n
CT534 t534 0 0.1f
M1968 t533 nw336 t534 0 nch w=1u l=180n
CT535 t535 0 0.1f
M1969 t534 nw366 t535 0 nch w=1u l=180n
M1970 t535 nen 0 0 nch w=1u l=180n
M1971 nw451 t529 vdd vdd pch w=2u l=180n
M1972 nw451 t529 0 0 nch w=1u l=180n
Cnw451 nw451 0 2f
M1973 nw452 nd14 vdd vdd pch w=2u l=180n
M1974 nw452 nw451 vdd vdd pch w=2u l=180n
CT536 t536 0 0.1f
M1975 nw452 nd14 t536 0 nch w=1u l=180n
M1976 t536 nw451 0 0 nch w=1u l=180n
Cnw452 nw452 0 2f
M1977 nw453 nd14 vdd vdd pch w=2u l=180n
M1978 nw453 nw452 vdd vdd pch w=2u l=180n
CT537 t537 0 0.1f
M1979 nw453 nd14 t537 0 nch w=1u l=180n
M1980 t537 nw452 0 0 nch w=1u l=180n
Cnw453 nw453 0 2f
M1981 nw454 nw451 vdd vdd pch w=2u l=180n
M1982 nw454 nw452 vdd vdd pch w=2u l=180n
CT538 t538 0 0.1f
M1983 nw454 nw451 t538 0 nch w=1u l=180n
M1984 t538 nw452 0 0 nch w=1u l=180n
Cnw454 nw454 0 2f
M1985 nw455 nw453 vdd vdd pch w=2u l=180n
M1986 nw455 nw454 vdd vdd pch w=2u l=180n
CT539 t539 0 0.1f
M1987 nw455 nw453 t539 0 nch w=1u l=180n
M1988 t539 nw454 0 0 nch w=1u l=180n
Cnw455 nw455 0 2f
CT540 t540 0 0.1f
M1989 t540 nw455 vdd vdd pch w=2u l=180n
M1990 t540 nw455 0 0 nch w=1u l=180n
M1991 nq14 t540 vdd vdd pch w=2u l=180n
M1992 nq14 t540 0 0 nch w=1u l=180n
Cnq14 nq14 0 2f
CT541 t541 0 0.1f
M1993 t541 nw72 vdd vdd pch w=2u l=180n
M1994 t541 nw362 vdd vdd pch w=2u l=180n
M1995 t541 nw216 vdd vdd pch w=2u l=180n
M1996 t541 nw364 vdd vdd pch w=2u l=180n
M1997 t541 nw336 vdd vdd pch w=2u l=180n
M1998 t541 nw366 vdd vdd pch w=2u l=180n
M1999 t541 nen vdd vdd pch w=2u l=180n
CT542 t542 0 0.1f
M2000 t541 nw72 t542 0 nch w=1u l=180n
CT543 t543 0 0.1f
M2001 t542 nw362 t543 0 nch w=1u l=180n
CT544 t544 0 0.1f
M2002 t543 nw216 t544 0 nch w=1u l=180n
CT545 t545 0 0.1f
M2003 t544 nw364 t545 0 nch w=1u l=180n
CT546 t546 0 0.1f
M2004 t545 nw336 t546 0 nch w=1u l=180n
CT547 t547 0 0.1f
M2005 t546 nw366 t547 0 nch w=1u l=180n
M2006 t547 nen 0 0 nch w=1u l=180n
M2007 nw457 t541 vdd vdd pch w=2u l=180n
M2008 nw457 t541 0 0 nch w=1u l=180n
Cnw457 nw457 0 2f
M2009 nw458 nd15 vdd vdd pch w=2u l=180n
M2010 nw458 nw457 vdd vdd pch w=2u l=180n
CT548 t548 0 0.1f
M2011 nw458 nd15 t548 0 nch w=1u l=180n
M2012 t548 nw457 0 0 nch w=1u l=180n
Cnw458 nw458 0 2f
M2013 nw459 nd15 vdd vdd pch w=2u l=180n
M2014 nw459 nw458 vdd vdd pch w=2u l=180n
CT549 t549 0 0.1f
M2015 nw459 nd15 t549 0 nch w=1u l=180n
M2016 t549 nw458 0 0 nch w=1u l=180n
Cnw459 nw459 0 2f
M2017 nw460 nw457 vdd vdd pch w=2u l=180n
M2018 nw460 nw458 vdd vdd pch w=2u l=180n
CT550 t550 0 0.1f
M2019 nw460 nw457 t550 0 nch w=1u l=180n
M2020 t550 nw458 0 0 nch w=1u l=180n
Cnw460 nw460 0 2f
M2021 nw461 nw459 vdd vdd pch w=2u l=180n
M2022 nw461 nw460 vdd vdd pch w=2u l=180n
CT551 t551 0 0.1f
M2023 nw461 nw459 t551 0 nch w=1u l=180n
M2024 t551 nw460 0 0 nch w=1u l=180n
Cnw461 nw461 0 2f
CT552 t552 0 0.1f
M2025 t552 nw461 vdd vdd pch w=2u l=180n
M2026 t552 nw461 0 0 nch w=1u l=180n
M2027 nq15 t552 vdd vdd pch w=2u l=180n
M2028 nq15 t552 0 0 nch w=1u l=180n
Cnq15 nq15 0 2f
CT553 t553 0 0.1f
M2029 t553 nw361 vdd vdd pch w=2u l=180n
M2030 t553 nw144 vdd vdd pch w=2u l=180n
M2031 t553 nw216 vdd vdd pch w=2u l=180n
M2032 t553 nw364 vdd vdd pch w=2u l=180n
M2033 t553 nw336 vdd vdd pch w=2u l=180n
M2034 t553 nw366 vdd vdd pch w=2u l=180n
M2035 t553 nen vdd vdd pch w=2u l=180n
CT554 t554 0 0.1f
M2036 t553 nw361 t554 0 nch w=1u l=180n
CT555 t555 0 0.1f
M2037 t554 nw144 t555 0 nch w=1u l=180n
CT556 t556 0 0.1f
M2038 t555 nw216 t556 0 nch w=1u l=180n
CT557 t557 0 0.1f
M2039 t556 nw364 t557 0 nch w=1u l=180n
CT558 t558 0 0.1f
M2040 t557 nw336 t558 0 nch w=1u l=180n
CT559 t559 0 0.1f
M2041 t558 nw366 t559 0 nch w=1u l=180n
M2042 t559 nen 0 0 nch w=1u l=180n
M2043 nw463 t553 vdd vdd pch w=2u l=180n
M2044 nw463 t553 0 0 nch w=1u l=180n
Cnw463 nw463 0 2f
M2045 nw464 nd16 vdd vdd pch w=2u l=180n
M2046 nw464 nw463 vdd vdd pch w=2u l=180n
CT560 t560 0 0.1f
M2047 nw464 nd16 t560 0 nch w=1u l=180n
M2048 t560 nw463 0 0 nch w=1u l=180n
Cnw464 nw464 0 2f
M2049 nw465 nd16 vdd vdd pch w=2u l=180n
M2050 nw465 nw464 vdd vdd pch w=2u l=180n
CT561 t561 0 0.1f
M2051 nw465 nd16 t561 0 nch w=1u l=180n
M2052 t561 nw464 0 0 nch w=1u l=180n
Cnw465 nw465 0 2f
M2053 nw466 nw463 vdd vdd pch w=2u l=180n
M2054 nw466 nw464 vdd vdd pch w=2u l=180n
CT562 t562 0 0.1f
M2055 nw466 nw463 t562 0 nch w=1u l=180n
M2056 t562 nw464 0 0 nch w=1u l=180n
Cnw466 nw466 0 2f
M2057 nw467 nw465 vdd vdd pch w=2u l=180n
M2058 nw467 nw466 vdd vdd pch w=2u l=180n
CT563 t563 0 0.1f
M2059 nw467 nw465 t563 0 nch w=1u l=180n
M2060 t563 nw466 0 0 nch w=1u l=180n
Cnw467 nw467 0 2f
CT564 t564 0 0.1f
M2061 t564 nw467 vdd vdd pch w=2u l=180n
M2062 t564 nw467 0 0 nch w=1u l=180n
M2063 nq16 t564 vdd vdd pch w=2u l=180n
M2064 nq16 t564 0 0 nch w=1u l=180n
Cnq16 nq16 0 2f
CT565 t565 0 0.1f
M2065 t565 nw72 vdd vdd pch w=2u l=180n
M2066 t565 nw144 vdd vdd pch w=2u l=180n
M2067 t565 nw216 vdd vdd pch w=2u l=180n
M2068 t565 nw364 vdd vdd pch w=2u l=180n
M2069 t565 nw336 vdd vdd pch w=2u l=180n
M2070 t565 nw366 vdd vdd pch w=2u l=180n
M2071 t565 nen vdd vdd pch w=2u l=180n
CT566 t566 0 0.1f
M2072 t565 nw72 t566 0 nch w=1u l=180n
CT567 t567 0 0.1f
M2073 t566 nw144 t567 0 nch w=1u l=180n
CT568 t568 0 0.1f
M2074 t567 nw216 t568 0 nch w=1u l=180n
CT569 t569 0 0.1f
M2075 t568 nw364 t569 0 nch w=1u l=180n
CT570 t570 0 0.1f
M2076 t569 nw336 t570 0 nch w=1u l=180n
CT571 t571 0 0.1f
M2077 t570 nw366 t571 0 nch w=1u l=180n
M2078 t571 nen 0 0 nch w=1u l=180n
M2079 nw469 t565 vdd vdd pch w=2u l=180n
M2080 nw469 t565 0 0 nch w=1u l=180n
Cnw469 nw469 0 2f
M2081 nw470 nd17 vdd vdd pch w=2u l=180n
M2082 nw470 nw469 vdd vdd pch w=2u l=180n
CT572 t572 0 0.1f
M2083 nw470 nd17 t572 0 nch w=1u l=180n
M2084 t572 nw469 0 0 nch w=1u l=180n
Cnw470 nw470 0 2f
M2085 nw471 nd17 vdd vdd pch w=2u l=180n
M2086 nw471 nw470 vdd vdd pch w=2u l=180n
CT573 t573 0 0.1f
M2087 nw471 nd17 t573 0 nch w=1u l=180n
M2088 t573 nw470 0 0 nch w=1u l=180n
Cnw471 nw471 0 2f
M2089 nw472 nw469 vdd vdd pch w=2u l=180n
M2090 nw472 nw470 vdd vdd pch w=2u l=180n
CT574 t574 0 0.1f
M2091 nw472 nw469 t574 0 nch w=1u l=180n
M2092 t574 nw470 0 0 nch w=1u l=180n
Cnw472 nw472 0 2f
M2093 nw473 nw471 vdd vdd pch w=2u l=180n
M2094 nw473 nw472 vdd vdd pch w=2u l=180n
CT575 t575 0 0.1f
M2095 nw473 nw471 t575 0 nch w=1u l=180n
M2096 t575 nw472 0 0 nch w=1u l=180n
Cnw473 nw473 0 2f
CT576 t576 0 0.1f
M2097 t576 nw473 vdd vdd pch w=2u l=180n
M2098 t576 nw473 0 0 nch w=1u l=180n
M2099 nq17 t576 vdd vdd pch w=2u l=180n
M2100 nq17 t576 0 0 nch w=1u l=180n
Cnq17 nq17 0 2f
CT577 t577 0 0.1f
M2101 t577 nw361 vdd vdd pch w=2u l=180n
M2102 t577 nw362 vdd vdd pch w=2u l=180n
M2103 t577 nw363 vdd vdd pch w=2u l=180n
M2104 t577 nw276 vdd vdd pch w=2u l=180n
M2105 t577 nw336 vdd vdd pch w=2u l=180n
M2106 t577 nw366 vdd vdd pch w=2u l=180n
M2107 t577 nen vdd vdd pch w=2u l=180n
CT578 t578 0 0.1f
M2108 t577 nw361 t578 0 nch w=1u l=180n
CT579 t579 0 0.1f
M2109 t578 nw362 t579 0 nch w=1u l=180n
CT580 t580 0 0.1f
M2110 t579 nw363 t580 0 nch w=1u l=180n
CT581 t581 0 0.1f
M2111 t580 nw276 t581 0 nch w=1u l=180n
CT582 t582 0 0.1f
M2112 t581 nw336 t582 0 nch w=1u l=180n
CT583 t583 0 0.1f
M2113 t582 nw366 t583 0 nch w=1u l=180n
M2114 t583 nen 0 0 nch w=1u l=180n
M2115 nw475 t577 vdd vdd pch w=2u l=180n
M2116 nw475 t577 0 0 nch w=1u l=180n
Cnw475 nw475 0 2f
M2117 nw476 nd18 vdd vdd pch w=2u l=180n
M2118 nw476 nw475 vdd vdd pch w=2u l=180n
CT584 t584 0 0.1f
M2119 nw476 nd18 t584 0 nch w=1u l=180n
M2120 t584 nw475 0 0 nch w=1u l=180n
Cnw476 nw476 0 2f
M2121 nw477 nd18 vdd vdd pch w=2u l=180n
M2122 nw477 nw476 vdd vdd pch w=2u l=180n
CT585 t585 0 0.1f
M2123 nw477 nd18 t585 0 nch w=1u l=180n
M2124 t585 nw476 0 0 nch w=1u l=180n
Cnw477 nw477 0 2f
M2125 nw478 nw475 vdd vdd pch w=2u l=180n
M2126 nw478 nw476 vdd vdd pch w=2u l=180n
CT586 t586 0 0.1f
M2127 nw478 nw475 t586 0 nch w=1u l=180n
M2128 t586 nw476 0 0 nch w=1u l=180n
Cnw478 nw478 0 2f
M2129 nw479 nw477 vdd vdd pch w=2u l=180n
M2130 nw479 nw478 vdd vdd pch w=2u l=180n
CT587 t587 0 0.1f
M2131 nw479 nw477 t587 0 nch w=1u l=180n
M2132 t587 nw478 0 0 nch w=1u l=180n
Cnw479 nw479 0 2f
CT588 t588 0 0.1f
M2133 t588 nw479 vdd vdd pch w=2u l=180n
M2134 t588 nw479 0 0 nch w=1u l=180n
M2135 nq18 t588 vdd vdd pch w=2u l=180n
M2136 nq18 t588 0 0 nch w=1u l=180n
Cnq18 nq18 0 2f
CT589 t589 0 0.1f
M2137 t589 nw72 vdd vdd pch w=2u l=180n
M2138 t589 nw362 vdd vdd pch w=2u l=180n
M2139 t589 nw363 vdd vdd pch w=2u l=180n
M2140 t589 nw276 vdd vdd pch w=2u l=180n
M2141 t589 nw336 vdd vdd pch w=2u l=180n
M2142 t589 nw366 vdd vdd pch w=2u l=180n
M2143 t589 nen vdd vdd pch w=2u l=180n
CT590 t590 0 0.1f
M2144 t589 nw72 t590 0 nch w=1u l=180n
CT591 t591 0 0.1f
M2145 t590 nw362 t591 0 nch w=1u l=180n
CT592 t592 0 0.1f
M2146 t591 nw363 t592 0 nch w=1u l=180n
CT593 t593 0 0.1f
M2147 t592 nw276 t593 0 nch w=1u l=180n
CT594 t594 0 0.1f
M2148 t593 nw336 t594 0 nch w=1u l=180n
CT595 t595 0 0.1f
M2149 t594 nw366 t595 0 nch w=1u l=180n
M2150 t595 nen 0 0 nch w=1u l=180n
M2151 nw481 t589 vdd vdd pch w=2u l=180n
M2152 nw481 t589 0 0 nch w=1u l=180n
Cnw481 nw481 0 2f
M2153 nw482 nd19 vdd vdd pch w=2u l=180n
M2154 nw482 nw481 vdd vdd pch w=2u l=180n
CT596 t596 0 0.1f
M2155 nw482 nd19 t596 0 nch w=1u l=180n
M2156 t596 nw481 0 0 nch w=1u l=180n
Cnw482 nw482 0 2f
M2157 nw483 nd19 vdd vdd pch w=2u l=180n
M2158 nw483 nw482 vdd vdd pch w=2u l=180n
CT597 t597 0 0.1f
M2159 nw483 nd19 t597 0 nch w=1u l=180n
M2160 t597 nw482 0 0 nch w=1u l=180n
Cnw483 nw483 0 2f
M2161 nw484 nw481 vdd vdd pch w=2u l=180n
M2162 nw484 nw482 vdd vdd pch w=2u l=180n
CT598 t598 0 0.1f
M2163 nw484 nw481 t598 0 nch w=1u l=180n
M2164 t598 nw482 0 0 nch w=1u l=180n
Cnw484 nw484 0 2f
M2165 nw485 nw483 vdd vdd pch w=2u l=180n
M2166 nw485 nw484 vdd vdd pch w=2u l=180n
CT599 t599 0 0.1f
M2167 nw485 nw483 t599 0 nch w=1u l=180n
M2168 t599 nw484 0 0 nch w=1u l=180n
Cnw485 nw485 0 2f
CT600 t600 0 0.1f
M2169 t600 nw485 vdd vdd pch w=2u l=180n
M2170 t600 nw485 0 0 nch w=1u l=180n
M2171 nq19 t600 vdd vdd pch w=2u l=180n
M2172 nq19 t600 0 0 nch w=1u l=180n
Cnq19 nq19 0 2f
CT601 t601 0 0.1f
M2173 t601 nw361 vdd vdd pch w=2u l=180n
M2174 t601 nw144 vdd vdd pch w=2u l=180n
M2175 t601 nw363 vdd vdd pch w=2u l=180n
M2176 t601 nw276 vdd vdd pch w=2u l=180n
M2177 t601 nw336 vdd vdd pch w=2u l=180n
M2178 t601 nw366 vdd vdd pch w=2u l=180n
M2179 t601 nen vdd vdd pch w=2u l=180n
CT602 t602 0 0.1f
M2180 t601 nw361 t602 0 nch w=1u l=180n
CT603 t603 0 0.1f
M2181 t602 nw144 t603 0 nch w=1u l=180n
CT604 t604 0 0.1f
M2182 t603 nw363 t604 0 nch w=1u l=180n
CT605 t605 0 0.1f
M2183 t604 nw276 t605 0 nch w=1u l=180n
CT606 t606 0 0.1f
M2184 t605 nw336 t606 0 nch w=1u l=180n
CT607 t607 0 0.1f
M2185 t606 nw366 t607 0 nch w=1u l=180n
M2186 t607 nen 0 0 nch w=1u l=180n
M2187 nw487 t601 vdd vdd pch w=2u l=180n
M2188 nw487 t601 0 0 nch w=1u l=180n
Cnw487 nw487 0 2f
M2189 nw488 nd20 vdd vdd pch w=2u l=180n
M2190 nw488 nw487 vdd vdd pch w=2u l=180n
CT608 t608 0 0.1f
M2191 nw488 nd20 t608 0 nch w=1u l=180n
M2192 t608 nw487 0 0 nch w=1u l=180n
Cnw488 nw488 0 2f
M2193 nw489 nd20 vdd vdd pch w=2u l=180n
M2194 nw489 nw488 vdd vdd pch w=2u l=180n
CT609 t609 0 0.1f
M2195 nw489 nd20 t609 0 nch w=1u l=180n
M2196 t609 nw488 0 0 nch w=1u l=180n
Cnw489 nw489 0 2f
M2197 nw490 nw487 vdd vdd pch w=2u l=180n
M2198 nw490 nw488 vdd vdd pch w=2u l=180n
CT610 t610 0 0.1f
M2199 nw490 nw487 t610 0 nch w=1u l=180n
M2200 t610 nw488 0 0 nch w=1u l=180n
Cnw490 nw490 0 2f
M2201 nw491 nw489 vdd vdd pch w=2u l=180n
M2202 nw491 nw490 vdd vdd pch w=2u l=180n
CT611 t611 0 0.1f
M2203 nw491 nw489 t611 0 nch w=1u l=180n
M2204 t611 nw490 0 0 nch w=1u l=180n
Cnw491 nw491 0 2f
CT612 t612 0 0.1f
M2205 t612 nw491 vdd vdd pch w=2u l=180n
M2206 t612 nw491 0 0 nch w=1u l=180n
M2207 nq20 t612 vdd vdd pch w=2u l=180n
M2208 nq20 t612 0 0 nch w=1u l=180n
Cnq20 nq20 0 2f
CT613 t613 0 0.1f
M2209 t613 nw72 vdd vdd pch w=2u l=180n
M2210 t613 nw144 vdd vdd pch w=2u l=180n
M2211 t613 nw363 vdd vdd pch w=2u l=180n
M2212 t613 nw276 vdd vdd pch w=2u l=180n
M2213 t613 nw336 vdd vdd pch w=2u l=180n
M2214 t613 nw366 vdd vdd pch w=2u l=180n
M2215 t613 nen vdd vdd pch w=2u l=180n
CT614 t614 0 0.1f
M2216 t613 nw72 t614 0 nch w=1u l=180n
CT615 t615 0 0.1f
M2217 t614 nw144 t615 0 nch w=1u l=180n
CT616 t616 0 0.1f
M2218 t615 nw363 t616 0 nch w=1u l=180n
CT617 t617 0 0.1f
M2219 t616 nw276 t617 0 nch w=1u l=180n
CT618 t618 0 0.1f
M2220 t617 nw336 t618 0 nch w=1u l=180n
CT619 t619 0 0.1f
M2221 t618 nw366 t619 0 nch w=1u l=180n
M2222 t619 nen 0 0 nch w=1u l=180n
M2223 nw493 t613 vdd vdd pch w=2u l=180n
M2224 nw493 t613 0 0 nch w=1u l=180n
Cnw493 nw493 0 2f
M2225 nw494 nd21 vdd vdd pch w=2u l=180n
M2226 nw494 nw493 vdd vdd pch w=2u l=180n
CT620 t620 0 0.1f
M2227 nw494 nd21 t620 0 nch w=1u l=180n
M2228 t620 nw493 0 0 nch w=1u l=180n
Cnw494 nw494 0 2f
M2229 nw495 nd21 vdd vdd pch w=2u l=180n
M2230 nw495 nw494 vdd vdd pch w=2u l=180n
CT621 t621 0 0.1f
M2231 nw495 nd21 t621 0 nch w=1u l=180n
M2232 t621 nw494 0 0 nch w=1u l=180n
Cnw495 nw495 0 2f
M2233 nw496 nw493 vdd vdd pch w=2u l=180n
M2234 nw496 nw494 vdd vdd pch w=2u l=180n
CT622 t622 0 0.1f
M2235 nw496 nw493 t622 0 nch w=1u l=180n
M2236 t622 nw494 0 0 nch w=1u l=180n
Cnw496 nw496 0 2f
M2237 nw497 nw495 vdd vdd pch w=2u l=180n
M2238 nw497 nw496 vdd vdd pch w=2u l=180n
CT623 t623 0 0.1f
M2239 nw497 nw495 t623 0 nch w=1u l=180n
M2240 t623 nw496 0 0 nch w=1u l=180n
Cnw497 nw497 0 2f
CT624 t624 0 0.1f
M2241 t624 nw497 vdd vdd pch w=2u l=180n
M2242 t624 nw497 0 0 nch w=1u l=180n
M2243 nq21 t624 vdd vdd pch w=2u l=180n
M2244 nq21 t624 0 0 nch w=1u l=180n
Cnq21 nq21 0 2f
CT625 t625 0 0.1f
M2245 t625 nw361 vdd vdd pch w=2u l=180n
M2246 t625 nw362 vdd vdd pch w=2u l=180n
M2247 t625 nw216 vdd vdd pch w=2u l=180n
M2248 t625 nw276 vdd vdd pch w=2u l=180n
M2249 t625 nw336 vdd vdd pch w=2u l=180n
M2250 t625 nw366 vdd vdd pch w=2u l=180n
M2251 t625 nen vdd vdd pch w=2u l=180n
CT626 t626 0 0.1f
M2252 t625 nw361 t626 0 nch w=1u l=180n
CT627 t627 0 0.1f
M2253 t626 nw362 t627 0 nch w=1u l=180n
CT628 t628 0 0.1f
M2254 t627 nw216 t628 0 nch w=1u l=180n
CT629 t629 0 0.1f
M2255 t628 nw276 t629 0 nch w=1u l=180n
CT630 t630 0 0.1f
M2256 t629 nw336 t630 0 nch w=1u l=180n
CT631 t631 0 0.1f
M2257 t630 nw366 t631 0 nch w=1u l=180n
M2258 t631 nen 0 0 nch w=1u l=180n
M2259 nw499 t625 vdd vdd pch w=2u l=180n
M2260 nw499 t625 0 0 nch w=1u l=180n
Cnw499 nw499 0 2f
M2261 nw500 nd22 vdd vdd pch w=2u l=180n
M2262 nw500 nw499 vdd vdd pch w=2u l=180n
CT632 t632 0 0.1f
M2263 nw500 nd22 t632 0 nch w=1u l=180n
M2264 t632 nw499 0 0 nch w=1u l=180n
Cnw500 nw500 0 2f
M2265 nw501 nd22 vdd vdd pch w=2u l=180n
M2266 nw501 nw500 vdd vdd pch w=2u l=180n
CT633 t633 0 0.1f
M2267 nw501 nd22 t633 0 nch w=1u l=180n
M2268 t633 nw500 0 0 nch w=1u l=180n
Cnw501 nw501 0 2f
M2269 nw502 nw499 vdd vdd pch w=2u l=180n
M2270 nw502 nw500 vdd vdd pch w=2u l=180n
CT634 t634 0 0.1f
M2271 nw502 nw499 t634 0 nch w=1u l=180n
M2272 t634 nw500 0 0 nch w=1u l=180n
Cnw502 nw502 0 2f
M2273 nw503 nw501 vdd vdd pch w=2u l=180n
M2274 nw503 nw502 vdd vdd pch w=2u l=180n
CT635 t635 0 0.1f
M2275 nw503 nw501 t635 0 nch w=1u l=180n
M2276 t635 nw502 0 0 nch w=1u l=180n
Cnw503 nw503 0 2f
CT636 t636 0 0.1f
M2277 t636 nw503 vdd vdd pch w=2u l=180n
M2278 t636 nw503 0 0 nch w=1u l=180n
M2279 nq22 t636 vdd vdd pch w=2u l=180n
M2280 nq22 t636 0 0 nch w=1u l=180n
Cnq22 nq22 0 2f
CT637 t637 0 0.1f
M2281 t637 nw72 vdd vdd pch w=2u l=180n
M2282 t637 nw362 vdd vdd pch w=2u l=180n
M2283 t637 nw216 vdd vdd pch w=2u l=180n
M2284 t637 nw276 vdd vdd pch w=2u l=180n
M2285 t637 nw336 vdd vdd pch w=2u l=180n
M2286 t637 nw366 vdd vdd pch w=2u l=180n
M2287 t637 nen vdd vdd pch w=2u l=180n
CT638 t638 0 0.1f
M2288 t637 nw72 t638 0 nch w=1u l=180n
CT639 t639 0 0.1f
M2289 t638 nw362 t639 0 nch w=1u l=180n
CT640 t640 0 0.1f
M2290 t639 nw216 t640 0 nch w=1u l=180n
CT641 t641 0 0.1f
M2291 t640 nw276 t641 0 nch w=1u l=180n
CT642 t642 0 0.1f
M2292 t641 nw336 t642 0 nch w=1u l=180n
CT643 t643 0 0.1f
M2293 t642 nw366 t643 0 nch w=1u l=180n
M2294 t643 nen 0 0 nch w=1u l=180n
M2295 nw505 t637 vdd vdd pch w=2u l=180n
M2296 nw505 t637 0 0 nch w=1u l=180n
Cnw505 nw505 0 2f
M2297 nw506 nd23 vdd vdd pch w=2u l=180n
M2298 nw506 nw505 vdd vdd pch w=2u l=180n
CT644 t644 0 0.1f
M2299 nw506 nd23 t644 0 nch w=1u l=180n
M2300 t644 nw505 0 0 nch w=1u l=180n
Cnw506 nw506 0 2f
M2301 nw507 nd23 vdd vdd pch w=2u l=180n
M2302 nw507 nw506 vdd vdd pch w=2u l=180n
CT645 t645 0 0.1f
M2303 nw507 nd23 t645 0 nch w=1u l=180n
M2304 t645 nw506 0 0 nch w=1u l=180n
Cnw507 nw507 0 2f
M2305 nw508 nw505 vdd vdd pch w=2u l=180n
M2306 nw508 nw506 vdd vdd pch w=2u l=180n
CT646 t646 0 0.1f
M2307 nw508 nw505 t646 0 nch w=1u l=180n
M2308 t646 nw506 0 0 nch w=1u l=180n
Cnw508 nw508 0 2f
M2309 nw509 nw507 vdd vdd pch w=2u l=180n
M2310 nw509 nw508 vdd vdd pch w=2u l=180n
CT647 t647 0 0.1f
M2311 nw509 nw507 t647 0 nch w=1u l=180n
M2312 t647 nw508 0 0 nch w=1u l=180n
Cnw509 nw509 0 2f
CT648 t648 0 0.1f
M2313 t648 nw509 vdd vdd pch w=2u l=180n
M2314 t648 nw509 0 0 nch w=1u l=180n
M2315 nq23 t648 vdd vdd pch w=2u l=180n
M2316 nq23 t648 0 0 nch w=1u l=180n
Cnq23 nq23 0 2f
CT649 t649 0 0.1f
M2317 t649 nw361 vdd vdd pch w=2u l=180n
M2318 t649 nw144 vdd vdd pch w=2u l=180n
M2319 t649 nw216 vdd vdd pch w=2u l=180n
M2320 t649 nw276 vdd vdd pch w=2u l=180n
M2321 t649 nw336 vdd vdd pch w=2u l=180n
M2322 t649 nw366 vdd vdd pch w=2u l=180n
M2323 t649 nen vdd vdd pch w=2u l=180n
CT650 t650 0 0.1f
M2324 t649 nw361 t650 0 nch w=1u l=180n
CT651 t651 0 0.1f
M2325 t650 nw144 t651 0 nch w=1u l=180n
CT652 t652 0 0.1f
M2326 t651 nw216 t652 0 nch w=1u l=180n
CT653 t653 0 0.1f
M2327 t652 nw276 t653 0 nch w=1u l=180n
CT654 t654 0 0.1f
M2328 t653 nw336 t654 0 nch w=1u l=180n
CT655 t655 0 0.1f
M2329 t654 nw366 t655 0 nch w=1u l=180n
M2330 t655 nen 0 0 nch w=1u l=180n
M2331 nw511 t649 vdd vdd pch w=2u l=180n
M2332 nw511 t649 0 0 nch w=1u l=180n
Cnw511 nw511 0 2f
M2333 nw512 nd24 vdd vdd pch w=2u l=180n
M2334 nw512 nw511 vdd vdd pch w=2u l=180n
CT656 t656 0 0.1f
M2335 nw512 nd24 t656 0 nch w=1u l=180n
M2336 t656 nw511 0 0 nch w=1u l=180n
Cnw512 nw512 0 2f
M2337 nw513 nd24 vdd vdd pch w=2u l=180n
M2338 nw513 nw512 vdd vdd pch w=2u l=180n
CT657 t657 0 0.1f
M2339 nw513 nd24 t657 0 nch w=1u l=180n
M2340 t657 nw512 0 0 nch w=1u l=180n
Cnw513 nw513 0 2f
M2341 nw514 nw511 vdd vdd pch w=2u l=180n
M2342 nw514 nw512 vdd vdd pch w=2u l=180n
CT658 t658 0 0.1f
M2343 nw514 nw511 t658 0 nch w=1u l=180n
M2344 t658 nw512 0 0 nch w=1u l=180n
Cnw514 nw514 0 2f
M2345 nw515 nw513 vdd vdd pch w=2u l=180n
M2346 nw515 nw514 vdd vdd pch w=2u l=180n
CT659 t659 0 0.1f
M2347 nw515 nw513 t659 0 nch w=1u l=180n
M2348 t659 nw514 0 0 nch w=1u l=180n
Cnw515 nw515 0 2f
CT660 t660 0 0.1f
M2349 t660 nw515 vdd vdd pch w=2u l=180n
M2350 t660 nw515 0 0 nch w=1u l=180n
M2351 nq24 t660 vdd vdd pch w=2u l=180n
M2352 nq24 t660 0 0 nch w=1u l=180n
Cnq24 nq24 0 2f
CT661 t661 0 0.1f
M2353 t661 nw72 vdd vdd pch w=2u l=180n
M2354 t661 nw144 vdd vdd pch w=2u l=180n
M2355 t661 nw216 vdd vdd pch w=2u l=180n
M2356 t661 nw276 vdd vdd pch w=2u l=180n
M2357 t661 nw336 vdd vdd pch w=2u l=180n
M2358 t661 nw366 vdd vdd pch w=2u l=180n
M2359 t661 nen vdd vdd pch w=2u l=180n
CT662 t662 0 0.1f
M2360 t661 nw72 t662 0 nch w=1u l=180n
CT663 t663 0 0.1f
M2361 t662 nw144 t663 0 nch w=1u l=180n
CT664 t664 0 0.1f
M2362 t663 nw216 t664 0 nch w=1u l=180n
CT665 t665 0 0.1f
M2363 t664 nw276 t665 0 nch w=1u l=180n
CT666 t666 0 0.1f
M2364 t665 nw336 t666 0 nch w=1u l=180n
CT667 t667 0 0.1f
M2365 t666 nw366 t667 0 nch w=1u l=180n
M2366 t667 nen 0 0 nch w=1u l=180n
M2367 nw517 t661 vdd vdd pch w=2u l=180n
M2368 nw517 t661 0 0 nch w=1u l=180n
Cnw517 nw517 0 2f
M2369 nw518 nd25 vdd vdd pch w=2u l=180n
M2370 nw518 nw517 vdd vdd pch w=2u l=180n
CT668 t668 0 0.1f
M2371 nw518 nd25 t668 0 nch w=1u l=180n
M2372 t668 nw517 0 0 nch w=1u l=180n
Cnw518 nw518 0 2f
M2373 nw519 nd25 vdd vdd pch w=2u l=180n
M2374 nw519 nw518 vdd vdd pch w=2u l=180n
CT669 t669 0 0.1f
M2375 nw519 nd25 t669 0 nch w=1u l=180n
M2376 t669 nw518 0 0 nch w=1u l=180n
Cnw519 nw519 0 2f
M2377 nw520 nw517 vdd vdd pch w=2u l=180n
M2378 nw520 nw518 vdd vdd pch w=2u l=180n
CT670 t670 0 0.1f
M2379 nw520 nw517 t670 0 nch w=1u l=180n
M2380 t670 nw518 0 0 nch w=1u l=180n
Cnw520 nw520 0 2f
M2381 nw521 nw519 vdd vdd pch w=2u l=180n
M2382 nw521 nw520 vdd vdd pch w=2u l=180n
CT671 t671 0 0.1f
M2383 nw521 nw519 t671 0 nch w=1u l=180n
M2384 t671 nw520 0 0 nch w=1u l=180n
Cnw521 nw521 0 2f
CT672 t672 0 0.1f
M2385 t672 nw521 vdd vdd pch w=2u l=180n
M2386 t672 nw521 0 0 nch w=1u l=180n
M2387 nq25 t672 vdd vdd pch w=2u l=180n
M2388 nq25 t672 0 0 nch w=1u l=180n
Cnq25 nq25 0 2f
CT673 t673 0 0.1f
M2389 t673 nw72 vdd vdd pch w=2u l=180n
M2390 t673 nw362 vdd vdd pch w=2u l=180n
M2391 t673 nw363 vdd vdd pch w=2u l=180n
M2392 t673 nw364 vdd vdd pch w=2u l=180n
M2393 t673 nw365 vdd vdd pch w=2u l=180n
M2394 t673 nw360 vdd vdd pch w=2u l=180n
M2395 t673 nen vdd vdd pch w=2u l=180n
CT674 t674 0 0.1f
M2396 t673 nw72 t674 0 nch w=1u l=180n
CT675 t675 0 0.1f
M2397 t674 nw362 t675 0 nch w=1u l=180n
CT676 t676 0 0.1f
M2398 t675 nw363 t676 0 nch w=1u l=180n
CT677 t677 0 0.1f
M2399 t676 nw364 t677 0 nch w=1u l=180n
CT678 t678 0 0.1f
M2400 t677 nw365 t678 0 nch w=1u l=180n
CT679 t679 0 0.1f
M2401 t678 nw360 t679 0 nch w=1u l=180n
M2402 t679 nen 0 0 nch w=1u l=180n
M2403 nw523 t673 vdd vdd pch w=2u l=180n
M2404 nw523 t673 0 0 nch w=1u l=180n
Cnw523 nw523 0 2f
M2405 nw524 nd26 vdd vdd pch w=2u l=180n
M2406 nw524 nw523 vdd vdd pch w=2u l=180n
CT680 t680 0 0.1f
M2407 nw524 nd26 t680 0 nch w=1u l=180n
M2408 t680 nw523 0 0 nch w=1u l=180n
Cnw524 nw524 0 2f
M2409 nw525 nd26 vdd vdd pch w=2u l=180n
M2410 nw525 nw524 vdd vdd pch w=2u l=180n
CT681 t681 0 0.1f
M2411 nw525 nd26 t681 0 nch w=1u l=180n
M2412 t681 nw524 0 0 nch w=1u l=180n
Cnw525 nw525 0 2f
M2413 nw526 nw523 vdd vdd pch w=2u l=180n
M2414 nw526 nw524 vdd vdd pch w=2u l=180n
CT682 t682 0 0.1f
M2415 nw526 nw523 t682 0 nch w=1u l=180n
M2416 t682 nw524 0 0 nch w=1u l=180n
Cnw526 nw526 0 2f
M2417 nw527 nw525 vdd vdd pch w=2u l=180n
M2418 nw527 nw526 vdd vdd pch w=2u l=180n
CT683 t683 0 0.1f
M2419 nw527 nw525 t683 0 nch w=1u l=180n
M2420 t683 nw526 0 0 nch w=1u l=180n
Cnw527 nw527 0 2f
CT684 t684 0 0.1f
M2421 t684 nw527 vdd vdd pch w=2u l=180n
M2422 t684 nw527 0 0 nch w=1u l=180n
M2423 nq26 t684 vdd vdd pch w=2u l=180n
M2424 nq26 t684 0 0 nch w=1u l=180n
Cnq26 nq26 0 2f
CT685 t685 0 0.1f
M2425 t685 nw361 vdd vdd pch w=2u l=180n
M2426 t685 nw144 vdd vdd pch w=2u l=180n
M2427 t685 nw363 vdd vdd pch w=2u l=180n
M2428 t685 nw364 vdd vdd pch w=2u l=180n
M2429 t685 nw365 vdd vdd pch w=2u l=180n
M2430 t685 nw360 vdd vdd pch w=2u l=180n
M2431 t685 nen vdd vdd pch w=2u l=180n
CT686 t686 0 0.1f
M2432 t685 nw361 t686 0 nch w=1u l=180n
CT687 t687 0 0.1f
M2433 t686 nw144 t687 0 nch w=1u l=180n
CT688 t688 0 0.1f
M2434 t687 nw363 t688 0 nch w=1u l=180n
CT689 t689 0 0.1f
M2435 t688 nw364 t689 0 nch w=1u l=180n
CT690 t690 0 0.1f
M2436 t689 nw365 t690 0 nch w=1u l=180n
CT691 t691 0 0.1f
M2437 t690 nw360 t691 0 nch w=1u l=180n
M2438 t691 nen 0 0 nch w=1u l=180n
M2439 nw529 t685 vdd vdd pch w=2u l=180n
M2440 nw529 t685 0 0 nch w=1u l=180n
Cnw529 nw529 0 2f
M2441 nw530 nd27 vdd vdd pch w=2u l=180n
M2442 nw530 nw529 vdd vdd pch w=2u l=180n
CT692 t692 0 0.1f
M2443 nw530 nd27 t692 0 nch w=1u l=180n
M2444 t692 nw529 0 0 nch w=1u l=180n
Cnw530 nw530 0 2f
M2445 nw531 nd27 vdd vdd pch w=2u l=180n
M2446 nw531 nw530 vdd vdd pch w=2u l=180n
CT693 t693 0 0.1f
M2447 nw531 nd27 t693 0 nch w=1u l=180n
M2448 t693 nw530 0 0 nch w=1u l=180n
Cnw531 nw531 0 2f
M2449 nw532 nw529 vdd vdd pch w=2u l=180n
M2450 nw532 nw530 vdd vdd pch w=2u l=180n
CT694 t694 0 0.1f
M2451 nw532 nw529 t694 0 nch w=1u l=180n
M2452 t694 nw530 0 0 nch w=1u l=180n
Cnw532 nw532 0 2f
M2453 nw533 nw531 vdd vdd pch w=2u l=180n
M2454 nw533 nw532 vdd vdd pch w=2u l=180n
CT695 t695 0 0.1f
M2455 nw533 nw531 t695 0 nch w=1u l=180n
M2456 t695 nw532 0 0 nch w=1u l=180n
Cnw533 nw533 0 2f
CT696 t696 0 0.1f
M2457 t696 nw533 vdd vdd pch w=2u l=180n
M2458 t696 nw533 0 0 nch w=1u l=180n
M2459 nq27 t696 vdd vdd pch w=2u l=180n
M2460 nq27 t696 0 0 nch w=1u l=180n
Cnq27 nq27 0 2f
CT697 t697 0 0.1f
M2461 t697 nw72 vdd vdd pch w=2u l=180n
M2462 t697 nw144 vdd vdd pch w=2u l=180n
M2463 t697 nw363 vdd vdd pch w=2u l=180n
M2464 t697 nw364 vdd vdd pch w=2u l=180n
M2465 t697 nw365 vdd vdd pch w=2u l=180n
M2466 t697 nw360 vdd vdd pch w=2u l=180n
M2467 t697 nen vdd vdd pch w=2u l=180n
CT698 t698 0 0.1f
M2468 t697 nw72 t698 0 nch w=1u l=180n
CT699 t699 0 0.1f
M2469 t698 nw144 t699 0 nch w=1u l=180n
CT700 t700 0 0.1f
M2470 t699 nw363 t700 0 nch w=1u l=180n
CT701 t701 0 0.1f
M2471 t700 nw364 t701 0 nch w=1u l=180n
CT702 t702 0 0.1f
M2472 t701 nw365 t702 0 nch w=1u l=180n
CT703 t703 0 0.1f
M2473 t702 nw360 t703 0 nch w=1u l=180n
M2474 t703 nen 0 0 nch w=1u l=180n
M2475 nw535 t697 vdd vdd pch w=2u l=180n
M2476 nw535 t697 0 0 nch w=1u l=180n
Cnw535 nw535 0 2f
M2477 nw536 nd28 vdd vdd pch w=2u l=180n
M2478 nw536 nw535 vdd vdd pch w=2u l=180n
CT704 t704 0 0.1f
M2479 nw536 nd28 t704 0 nch w=1u l=180n
M2480 t704 nw535 0 0 nch w=1u l=180n
Cnw536 nw536 0 2f
M2481 nw537 nd28 vdd vdd pch w=2u l=180n
M2482 nw537 nw536 vdd vdd pch w=2u l=180n
CT705 t705 0 0.1f
M2483 nw537 nd28 t705 0 nch w=1u l=180n
M2484 t705 nw536 0 0 nch w=1u l=180n
Cnw537 nw537 0 2f
M2485 nw538 nw535 vdd vdd pch w=2u l=180n
M2486 nw538 nw536 vdd vdd pch w=2u l=180n
CT706 t706 0 0.1f
M2487 nw538 nw535 t706 0 nch w=1u l=180n
M2488 t706 nw536 0 0 nch w=1u l=180n
Cnw538 nw538 0 2f
M2489 nw539 nw537 vdd vdd pch w=2u l=180n
M2490 nw539 nw538 vdd vdd pch w=2u l=180n
CT707 t707 0 0.1f
M2491 nw539 nw537 t707 0 nch w=1u l=180n
M2492 t707 nw538 0 0 nch w=1u l=180n
Cnw539 nw539 0 2f
CT708 t708 0 0.1f
M2493 t708 nw539 vdd vdd pch w=2u l=180n
M2494 t708 nw539 0 0 nch w=1u l=180n
M2495 nq28 t708 vdd vdd pch w=2u l=180n
M2496 nq28 t708 0 0 nch w=1u l=180n
Cnq28 nq28 0 2f
CT709 t709 0 0.1f
M2497 t709 nw361 vdd vdd pch w=2u l=180n
M2498 t709 nw362 vdd vdd pch w=2u l=180n
M2499 t709 nw216 vdd vdd pch w=2u l=180n
M2500 t709 nw364 vdd vdd pch w=2u l=180n
M2501 t709 nw365 vdd vdd pch w=2u l=180n
M2502 t709 nw360 vdd vdd pch w=2u l=180n
M2503 t709 nen vdd vdd pch w=2u l=180n
CT710 t710 0 0.1f
M2504 t709 nw361 t710 0 nch w=1u l=180n
CT711 t711 0 0.1f
M2505 t710 nw362 t711 0 nch w=1u l=180n
CT712 t712 0 0.1f
M2506 t711 nw216 t712 0 nch w=1u l=180n
CT713 t713 0 0.1f
M2507 t712 nw364 t713 0 nch w=1u l=180n
CT714 t714 0 0.1f
M2508 t713 nw365 t714 0 nch w=1u l=180n
CT715 t715 0 0.1f
M2509 t714 nw360 t715 0 nch w=1u l=180n
M2510 t715 nen 0 0 nch w=1u l=180n
M2511 nw541 t709 vdd vdd pch w=2u l=180n
M2512 nw541 t709 0 0 nch w=1u l=180n
Cnw541 nw541 0 2f
M2513 nw542 nd29 vdd vdd pch w=2u l=180n
M2514 nw542 nw541 vdd vdd pch w=2u l=180n
CT716 t716 0 0.1f
M2515 nw542 nd29 t716 0 nch w=1u l=180n
M2516 t716 nw541 0 0 nch w=1u l=180n
Cnw542 nw542 0 2f
M2517 nw543 nd29 vdd vdd pch w=2u l=180n
M2518 nw543 nw542 vdd vdd pch w=2u l=180n
CT717 t717 0 0.1f
M2519 nw543 nd29 t717 0 nch w=1u l=180n
M2520 t717 nw542 0 0 nch w=1u l=180n
Cnw543 nw543 0 2f
M2521 nw544 nw541 vdd vdd pch w=2u l=180n
M2522 nw544 nw542 vdd vdd pch w=2u l=180n
CT718 t718 0 0.1f
M2523 nw544 nw541 t718 0 nch w=1u l=180n
M2524 t718 nw542 0 0 nch w=1u l=180n
Cnw544 nw544 0 2f
M2525 nw545 nw543 vdd vdd pch w=2u l=180n
M2526 nw545 nw544 vdd vdd pch w=2u l=180n
CT719 t719 0 0.1f
M2527 nw545 nw543 t719 0 nch w=1u l=180n
M2528 t719 nw544 0 0 nch w=1u l=180n
Cnw545 nw545 0 2f
CT720 t720 0 0.1f
M2529 t720 nw545 vdd vdd pch w=2u l=180n
M2530 t720 nw545 0 0 nch w=1u l=180n
M2531 nq29 t720 vdd vdd pch w=2u l=180n
M2532 nq29 t720 0 0 nch w=1u l=180n
Cnq29 nq29 0 2f
CT721 t721 0 0.1f
M2533 t721 nw72 vdd vdd pch w=2u l=180n
M2534 t721 nw362 vdd vdd pch w=2u l=180n
M2535 t721 nw216 vdd vdd pch w=2u l=180n
M2536 t721 nw364 vdd vdd pch w=2u l=180n
M2537 t721 nw365 vdd vdd pch w=2u l=180n
M2538 t721 nw360 vdd vdd pch w=2u l=180n
M2539 t721 nen vdd vdd pch w=2u l=180n
CT722 t722 0 0.1f
M2540 t721 nw72 t722 0 nch w=1u l=180n
CT723 t723 0 0.1f
M2541 t722 nw362 t723 0 nch w=1u l=180n
CT724 t724 0 0.1f
M2542 t723 nw216 t724 0 nch w=1u l=180n
CT725 t725 0 0.1f
M2543 t724 nw364 t725 0 nch w=1u l=180n
CT726 t726 0 0.1f
M2544 t725 nw365 t726 0 nch w=1u l=180n
CT727 t727 0 0.1f
M2545 t726 nw360 t727 0 nch w=1u l=180n
M2546 t727 nen 0 0 nch w=1u l=180n
M2547 nw547 t721 vdd vdd pch w=2u l=180n
M2548 nw547 t721 0 0 nch w=1u l=180n
Cnw547 nw547 0 2f
M2549 nw548 nd30 vdd vdd pch w=2u l=180n
M2550 nw548 nw547 vdd vdd pch w=2u l=180n
CT728 t728 0 0.1f
M2551 nw548 nd30 t728 0 nch w=1u l=180n
M2552 t728 nw547 0 0 nch w=1u l=180n
Cnw548 nw548 0 2f
M2553 nw549 nd30 vdd vdd pch w=2u l=180n
M2554 nw549 nw548 vdd vdd pch w=2u l=180n
CT729 t729 0 0.1f
M2555 nw549 nd30 t729 0 nch w=1u l=180n
M2556 t729 nw548 0 0 nch w=1u l=180n
Cnw549 nw549 0 2f
M2557 nw550 nw547 vdd vdd pch w=2u l=180n
M2558 nw550 nw548 vdd vdd pch w=2u l=180n
CT730 t730 0 0.1f
M2559 nw550 nw547 t730 0 nch w=1u l=180n
M2560 t730 nw548 0 0 nch w=1u l=180n
Cnw550 nw550 0 2f
M2561 nw551 nw549 vdd vdd pch w=2u l=180n
M2562 nw551 nw550 vdd vdd pch w=2u l=180n
CT731 t731 0 0.1f
M2563 nw551 nw549 t731 0 nch w=1u l=180n
M2564 t731 nw550 0 0 nch w=1u l=180n
Cnw551 nw551 0 2f
CT732 t732 0 0.1f
M2565 t732 nw551 vdd vdd pch w=2u l=180n
M2566 t732 nw551 0 0 nch w=1u l=180n
M2567 nq30 t732 vdd vdd pch w=2u l=180n
M2568 nq30 t732 0 0 nch w=1u l=180n
Cnq30 nq30 0 2f
CT733 t733 0 0.1f
M2569 t733 nw361 vdd vdd pch w=2u l=180n
M2570 t733 nw144 vdd vdd pch w=2u l=180n
M2571 t733 nw216 vdd vdd pch w=2u l=180n
M2572 t733 nw364 vdd vdd pch w=2u l=180n
M2573 t733 nw365 vdd vdd pch w=2u l=180n
M2574 t733 nw360 vdd vdd pch w=2u l=180n
M2575 t733 nen vdd vdd pch w=2u l=180n
CT734 t734 0 0.1f
M2576 t733 nw361 t734 0 nch w=1u l=180n
CT735 t735 0 0.1f
M2577 t734 nw144 t735 0 nch w=1u l=180n
CT736 t736 0 0.1f
M2578 t735 nw216 t736 0 nch w=1u l=180n
CT737 t737 0 0.1f
M2579 t736 nw364 t737 0 nch w=1u l=180n
CT738 t738 0 0.1f
M2580 t737 nw365 t738 0 nch w=1u l=180n
CT739 t739 0 0.1f
M2581 t738 nw360 t739 0 nch w=1u l=180n
M2582 t739 nen 0 0 nch w=1u l=180n
M2583 nw553 t733 vdd vdd pch w=2u l=180n
M2584 nw553 t733 0 0 nch w=1u l=180n
Cnw553 nw553 0 2f
M2585 nw554 nd31 vdd vdd pch w=2u l=180n
M2586 nw554 nw553 vdd vdd pch w=2u l=180n
CT740 t740 0 0.1f
M2587 nw554 nd31 t740 0 nch w=1u l=180n
M2588 t740 nw553 0 0 nch w=1u l=180n
Cnw554 nw554 0 2f
M2589 nw555 nd31 vdd vdd pch w=2u l=180n
M2590 nw555 nw554 vdd vdd pch w=2u l=180n
CT741 t741 0 0.1f
M2591 nw555 nd31 t741 0 nch w=1u l=180n
M2592 t741 nw554 0 0 nch w=1u l=180n
Cnw555 nw555 0 2f
M2593 nw556 nw553 vdd vdd pch w=2u l=180n
M2594 nw556 nw554 vdd vdd pch w=2u l=180n
CT742 t742 0 0.1f
M2595 nw556 nw553 t742 0 nch w=1u l=180n
M2596 t742 nw554 0 0 nch w=1u l=180n
Cnw556 nw556 0 2f
M2597 nw557 nw555 vdd vdd pch w=2u l=180n
M2598 nw557 nw556 vdd vdd pch w=2u l=180n
CT743 t743 0 0.1f
M2599 nw557 nw555 t743 0 nch w=1u l=180n
M2600 t743 nw556 0 0 nch w=1u l=180n
Cnw557 nw557 0 2f
CT744 t744 0 0.1f
M2601 t744 nw557 vdd vdd pch w=2u l=180n
M2602 t744 nw557 0 0 nch w=1u l=180n
M2603 nq31 t744 vdd vdd pch w=2u l=180n
M2604 nq31 t744 0 0 nch w=1u l=180n
Cnq31 nq31 0 2f
.model nch NMOS (vto=0.45 kp=200u lambda=0.05)
.model pch PMOS (vto=-0.45 kp=100u lambda=0.05)
* outputs: nq0 nq1 nq2 nq3 nq4 nq5 nq6 nq7 nq8 nq9 nq10 nq11 nq12 nq13 nq14 nq15 nq16 nq17 nq18 nq19 nq20 nq21 nq22 nq23 nq24 nq25 nq26 nq27 nq28 nq29 nq30 nq31
.end
